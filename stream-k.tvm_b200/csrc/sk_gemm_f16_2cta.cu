// fp16 NT Stream-K GEMM with CTA pairs (tcgen05 cta_group::2) for large problems.
//
// Same persistent Stream-K structure as sk_gemm_f16.cu (it stands in for the same
// reference kernels, streamk_fp16.py:116-373), but the scheduling unit is a cluster of
// two CTAs on one TPC that computes a 256 x 256 tile: each CTA loads its own 128 rows of
// A and its own 128 rows of B (half of the tile's columns) per K step, one thread of the
// leader CTA issues a 256 x 256 x 16 UMMA that reads both CTAs' shared memory, and each
// CTA ends up with its 128 x 256 half of the accumulator in its own TMEM.  Per flop a CTA
// pulls 2/3 of the bytes the single-CTA kernel does, so the same shared-memory budget
// covers 1.5x the load latency.  No load is multicast: each CTA fetches what it needs.
//
// Roles per CTA as in sk_gemm_f16.cu, but with eight epilogue warps (two per TMEM lane quadrant,
// splitting a tile's columns): draining a 128 x 256 accumulator is a latency chain per warp
// (TMEM load, convert, staging store, proxy fence, TMA store), and with tensor memory full of
// accumulators every microsecond of drain at a unit boundary is a microsecond without MMAs.
// The MMA warp of the second CTA only takes part in the tensor-memory allocation.
#include "sk_common.cuh"
#include "sk_epilogue.cuh"

namespace {

using namespace skptx;

constexpr int BM = SK_BM;            // rows per CTA
constexpr int BN = 256;              // tile columns (both CTAs see all of them in TMEM)
constexpr int BK = 64;
constexpr int A_STAGE_BYTES = BM * BK * 2;         // 16 KB
constexpr int B_STAGE_BYTES = (BN / 2) * BK * 2;   // 16 KB: this CTA's half of the B tile
constexpr int KG = 2;                  // K steps that share a pipeline stage (one barrier round trip)
constexpr int STAGES = 3;              // 3 x 2 x 32 KB = 192 KB
constexpr int EPI_WARPS = 8;
constexpr int NUM_THREADS = 64 + 32 * EPI_WARPS;   // warp 0 producer, warp 1 MMA issuer, warps 2..9 epilogue
constexpr int TMEM_COLS = 512;
constexpr int PIPE_BYTES = STAGES * KG * (A_STAGE_BYTES + B_STAGE_BYTES);
constexpr int CTRL_BYTES = 512;
constexpr int SMEM_BYTES = PIPE_BYTES + 1024 + CTRL_BYTES + 512 + SK_CSTAGE_BYTES;   // ... + TMA-store staging
static_assert(SMEM_BYTES <= 232448, "shared memory budget");

// Wide units (256 x 512: two column-adjacent tiles that share every A stage, one accumulator
// buffer each): a ring of its own in the same shared memory, one K step per stage.
constexpr int WSTAGES = 4;
constexpr int W_STAGE_BYTES = A_STAGE_BYTES + 2 * B_STAGE_BYTES;   // 48 KB: A | B of half 0 | B of half 1
static_assert(WSTAGES * W_STAGE_BYTES <= PIPE_BYTES, "the wide ring lives in the pipeline's memory");

struct Ctrl {
  uint64_t full[STAGES];      // used in the leader CTA: both CTAs' loads complete here
  uint64_t empty[STAGES];     // one per CTA, released by the leader's multicast commit
  uint64_t fullw[WSTAGES];    // the same pair for the wide ring
  uint64_t emptyw[WSTAGES];
  uint64_t tmem_full[2];      // one per CTA, multicast commit
  uint64_t tmem_empty[2];     // used in the leader CTA: one arrival per epilogue warp of both CTAs
  uint32_t tmem_base;
  uint32_t abort;
  uint32_t bcast;
  uint32_t ok[2];
  SkPending pend[2];
};
static_assert(sizeof(Ctrl) <= CTRL_BYTES, "Ctrl must fit its reserved space");

// OUT_GATHER: the fused all-gather (sk_gemm_f16_gather): the epilogue also writes every piece of
// C into the peer GPUs' matrices named by `peer_set`.  OUT_SCATTER: the fused reduce-scatter
// (sk_gemm_f16_scatter): the product is a partial sum over this GPU's share of K; every tile
// (whole tiles only: the data-parallel schedule) leaves as fp32 into the receive slot of the
// GPU that owns its column block, and nothing is written to C.
constexpr int OUT_PLAIN = 0, OUT_GATHER = 1, OUT_SCATTER = 2;

template <int OUT>
__global__ void __launch_bounds__(NUM_THREADS, 1)
sk_gemm_f16_2cta_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                        const __grid_constant__ CUtensorMap tmC, __half* __restrict__ C, const SkParams p,
                        const __grid_constant__ SkPeers peer_set) {
  constexpr bool PEERS = OUT == OUT_GATHER;
  const SkPeers* peers = PEERS ? &peer_set : nullptr;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw_addr);
  const uint32_t sA = base;
  const uint32_t sB = base + STAGES * KG * A_STAGE_BYTES;
  Ctrl* ctrl = reinterpret_cast<Ctrl*>(smem + PIPE_BYTES);
  volatile uint32_t* abort_flag = &ctrl->abort;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int rank = static_cast<int>(cluster_ctarank());   // 0 = leader of the pair
  const int unit = blockIdx.x >> 1;                        // the pair's index in the schedule
  const SkSched& s = p.sched;
  if (threadIdx.x == 0) {
    sk_trace(p, 0);
    griddep_launch_dependents();   // the next kernel of the stream may begin its own start-up
  }

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) {
      mbar_init(smem_u32(&ctrl->full[i]), 1);
      mbar_init(smem_u32(&ctrl->empty[i]), 1);
    }
    for (int i = 0; i < WSTAGES; ++i) {
      mbar_init(smem_u32(&ctrl->fullw[i]), 1);
      mbar_init(smem_u32(&ctrl->emptyw[i]), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&ctrl->tmem_full[i]), 1);
      mbar_init(smem_u32(&ctrl->tmem_empty[i]), 2 * EPI_WARPS);
    }
    ctrl->abort = 0u;
    ctrl->bcast = 0u;
    ctrl->pend[0].tile = -1;
    ctrl->pend[1].tile = -1;
    fence_mbar_init();
    fence_proxy_async_smem();
    prefetch_tensormap(&tmA);
    prefetch_tensormap(&tmB);
    if (OUT != OUT_PLAIN)
      for (int i = 0; i < peer_set.n; ++i) prefetch_tensormap(&peer_set.tm[i]);
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(&ctrl->tmem_base), TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();   // the partner's barriers are initialised before anyone signals them
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&ctrl->tmem_base);
  if (threadIdx.x == 0) sk_trace(p, 1);
  // global memory is the previous kernel's until it has completed (no-op without SK_FLAG_PDL)
  griddep_wait();

  if (warp == 0) {
    // ------------------------------------------------------------- producer (both CTAs)
    if (lane == 0) {
      SkCursor cur;
      sk_cursor_init(s, unit, cur);
      SkSeg seg;
      int stage = 0;
      uint32_t ph = 0;
      bool ok = true;
      bool traced = false;
      const uint32_t full0_leader = mapa_shared(smem_u32(&ctrl->full[0]), 0);
      const uint32_t full0 = smem_u32(&ctrl->full[0]), empty0 = smem_u32(&ctrl->empty[0]);
      while (ok && sk_next(s, unit, cur, seg)) {
        int tr, tc;
        sk_tile_mn(s, seg.tile, tr, tc);
        const int a_row0 = (tr * 2 + rank) * BM;          // this CTA's 128 rows of A
        const int b_row0 = tc * p.bn + rank * (p.bn / 2);   // this CTA's half of the tile's rows of B
        for (int k = seg.k0; k < seg.k1;) {
          const int n = (seg.k1 - k) < KG ? (seg.k1 - k) : KG;
          if (!sk_wait_bar(empty0 + 8u * stage, ph ^ 1u, abort_flag, p, stage, 0)) {
            ok = false;
            break;
          }
          // Both CTAs' loads complete on the leader's barrier; the leader expects all of them.
          const uint32_t full_leader = full0_leader + 8u * stage;
          if (rank == 0) mbar_arrive_expect_tx(full0 + 8u * stage, n * 2 * (A_STAGE_BYTES + p.col_tx_bytes));
          for (int j = 0; j < n; ++j) {
            tma_load_2d_pair(sA + (stage * KG + j) * A_STAGE_BYTES, &tmA, full_leader, (k + j) * BK, a_row0);
            tma_load_2d_pair(sB + (stage * KG + j) * B_STAGE_BYTES, &tmB, full_leader, (k + j) * BK, b_row0);
          }
          k += n;
          if (++stage == STAGES) { stage = 0; ph ^= 1u; }
          if (!traced) { sk_trace(p, 2); traced = true; }
        }
      }
      if (ok && p.wide_units > 0) {
        // ---- wide units.  First let the tiles' last stages drain: the wide ring reuses their memory.
        for (int i = 0; i < STAGES && ok; ++i) {
          ok = sk_wait_bar(empty0 + 8u * stage, ph ^ 1u, abort_flag, p, stage, 0);
          if (++stage == STAGES) { stage = 0; ph ^= 1u; }
        }
        const uint32_t fullw0_leader = mapa_shared(smem_u32(&ctrl->fullw[0]), 0);
        const uint32_t fullw0 = smem_u32(&ctrl->fullw[0]), emptyw0 = smem_u32(&ctrl->emptyw[0]);
        int ws = 0;
        uint32_t wph = 0;
        for (int u = unit; ok && u < p.wide_units; u += s.grid) {
          int tm, tnw;
          sk_raster_mn(s, u, tm, tnw);
          const int a_row0 = (tm * 2 + rank) * BM;
          const int b_row0 = tnw * (2 * BN) + rank * (BN / 2);   // half 0; half 1 is BN rows further
          for (int k = 0; k < s.iters_per_tile; ++k) {
            if (!sk_wait_bar(emptyw0 + 8u * ws, wph ^ 1u, abort_flag, p, 8 + ws, 0)) {
              ok = false;
              break;
            }
            const uint32_t dst = base + ws * W_STAGE_BYTES;
            const uint32_t full_leader = fullw0_leader + 8u * ws;
            if (rank == 0) mbar_arrive_expect_tx(fullw0 + 8u * ws, 2 * W_STAGE_BYTES);
            tma_load_2d_pair(dst, &tmA, full_leader, k * BK, a_row0);
            tma_load_2d_pair(dst + A_STAGE_BYTES, &tmB, full_leader, k * BK, b_row0);
            tma_load_2d_pair(dst + A_STAGE_BYTES + B_STAGE_BYTES, &tmB, full_leader, k * BK, b_row0 + BN);
            if (++ws == WSTAGES) { ws = 0; wph ^= 1u; }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------- MMA issuer (leader only)
    if (lane == 0 && rank == 0) {
      SkCursor cur;
      sk_cursor_init(s, unit, cur);
      SkSeg seg;
      int stage = 0;
      uint32_t ph = 0;
      uint32_t nseg = 0;
      bool ok = true;
      const uint64_t desc_hi = umma_desc_sw128_hi(16, 1024);
      const uint32_t a_lo0 = umma_desc_lo(sA), b_lo0 = umma_desc_lo(sB);
      const uint32_t idesc = p.idesc;
      const uint32_t full0 = smem_u32(&ctrl->full[0]), empty0 = smem_u32(&ctrl->empty[0]);
      while (ok && sk_next(s, unit, cur, seg)) {
        const uint32_t buf = nseg & 1u;
        const uint32_t acc_ph = (nseg >> 1) & 1u;
        if (!sk_wait_bar(smem_u32(&ctrl->tmem_empty[buf]), acc_ph ^ 1u, abort_flag, p, 16 + buf, 1))
          break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * BN;
        uint32_t accumulate = 0u;
        for (int k = seg.k0; k < seg.k1;) {
          const int n = (seg.k1 - k) < KG ? (seg.k1 - k) : KG;
          if (!sk_wait_bar(full0 + 8u * stage, ph, abort_flag, p, 32 + stage, 1)) {
            ok = false;
            break;
          }
          tc_fence_after();
          if (nseg == 0 && k == seg.k0) sk_trace(p, 3);
          for (int j = 0; j < n; ++j) {
            const uint32_t a_lo = a_lo0 + (stage * KG + j) * (A_STAGE_BYTES >> 4);
            const uint32_t b_lo = b_lo0 + (stage * KG + j) * (B_STAGE_BYTES >> 4);
#pragma unroll
            for (int kk = 0; kk < BK / 16; ++kk) {
              umma_f16_ss_pair(d_tmem, desc_hi | (a_lo + kk * 2), desc_hi | (b_lo + kk * 2), idesc, accumulate);
              accumulate = 1u;
            }
          }
          umma_commit_pair(empty0 + 8u * stage);   // frees the stage in both CTAs
          k += n;
          if (++stage == STAGES) { stage = 0; ph ^= 1u; }
        }
        if (!ok) break;
        umma_commit_pair(smem_u32(&ctrl->tmem_full[buf]));   // accumulator ready in both CTAs
        ++nseg;
      }
      if (ok && p.wide_units > 0) {
        // ---- wide units: every A stage feeds two accumulators (25 % fewer bytes into the SM
        // per flop, which is what bounds this kernel and what costs it power)
        const uint32_t fullw0 = smem_u32(&ctrl->fullw[0]), emptyw0 = smem_u32(&ctrl->emptyw[0]);
        const uint32_t w_lo0 = umma_desc_lo(base);
        int ws = 0;
        uint32_t wph = 0;
        for (int u = unit; ok && u < p.wide_units; u += s.grid) {
          const uint32_t buf0 = nseg & 1u, buf1 = buf0 ^ 1u;
          const uint32_t empty1 = smem_u32(&ctrl->tmem_empty[buf1]);
          const uint32_t empty1_ph = (((nseg + 1) >> 1) & 1u) ^ 1u;
          if (!sk_wait_bar(smem_u32(&ctrl->tmem_empty[buf0]), ((nseg >> 1) & 1u) ^ 1u, abort_flag, p, 16 + buf0, 1)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t d0 = tmem_base + buf0 * BN, d1 = tmem_base + buf1 * BN;
          // The epilogue drains the first half's buffer, then the second's.  The first half
          // starts as soon as its buffer is free and may run up to WSTAGES - 1 K steps ahead of
          // the second (the stages stay held until the second half has read them too), so the
          // second buffer's drain overlaps the start of this unit.  Once the second half may
          // run it catches up to within `lag` K steps (a held stage is a stage the producer
          // cannot refill) and stays that far behind: the first half then finishes `lag` steps
          // early, hands its accumulator to the epilogue at once, and its drain runs under the
          // second half's last MMAs instead of after them.
          const int I = s.iters_per_tile;
          const int lag = p.wide_lag;
          int k0 = 0, k1 = 0;          // next K step of the first / second half
          int ws1 = ws;                // stage of K step k1 (ws is the stage of k0)
          bool h1_ready = false;
          while (ok && k1 < I) {
            if (k0 < I && (h1_ready ? k0 - k1 <= lag : k0 - k1 < WSTAGES - 1)) {
              if (!sk_wait_bar(fullw0 + 8u * ws, wph, abort_flag, p, 40 + ws, 1)) {
                ok = false;
                break;
              }
              tc_fence_after();
              const uint32_t a_lo = w_lo0 + ws * (W_STAGE_BYTES >> 4);
              const uint32_t b_lo = a_lo + (A_STAGE_BYTES >> 4);
#pragma unroll
              for (int kk = 0; kk < BK / 16; ++kk)
                umma_f16_ss_pair(d0, desc_hi | (a_lo + kk * 2), desc_hi | (b_lo + kk * 2), idesc,
                                 (k0 | kk) ? 1u : 0u);
              ++k0;
              if (++ws == WSTAGES) { ws = 0; wph ^= 1u; }
              if (k0 == I) umma_commit_pair(smem_u32(&ctrl->tmem_full[buf0]));   // first half complete
            }
            if (!h1_ready) {
              if (mbar_try_wait(empty1, empty1_ph, 0u)) {
                h1_ready = true;
              } else if (k0 == I || k0 - k1 >= WSTAGES - 1) {   // cannot run further ahead: wait
                if (!sk_wait_bar(empty1, empty1_ph, abort_flag, p, 16 + buf1, 1)) {
                  ok = false;
                  break;
                }
                h1_ready = true;
              }
              if (h1_ready) tc_fence_after();
            }
            if (h1_ready && k1 < k0 && (k0 - k1 > lag || k0 == I)) {
              const uint32_t a_lo = w_lo0 + ws1 * (W_STAGE_BYTES >> 4);
              const uint32_t b_lo = a_lo + ((A_STAGE_BYTES + B_STAGE_BYTES) >> 4);
#pragma unroll
              for (int kk = 0; kk < BK / 16; ++kk)
                umma_f16_ss_pair(d1, desc_hi | (a_lo + kk * 2), desc_hi | (b_lo + kk * 2), idesc,
                                 (k1 | kk) ? 1u : 0u);
              umma_commit_pair(emptyw0 + 8u * ws1);   // both halves have read the stage
              ++k1;
              if (++ws1 == WSTAGES) ws1 = 0;
            }
          }
          if (!ok) break;
          umma_commit_pair(smem_u32(&ctrl->tmem_full[buf1]));
          nseg += 2;
        }
      }
      sk_trace(p, 4);
    }
  } else {
    // ------------------------------------------------------------- epilogue (both CTAs)
    const uint32_t cstage = p.c_tma ? smem_u32(ctrl) + 1024u : 0u;
    const uint32_t tmem_full0 = smem_u32(&ctrl->tmem_full[0]);
    const uint32_t tmem_empty0 = mapa_shared(smem_u32(&ctrl->tmem_empty[0]), 0);
    uint32_t nseg = 0;
    if constexpr (OUT == OUT_SCATTER) {
      // ---- fused reduce-scatter: whole tiles, fp32, each to the owner of its column block
      const int q = warp & 3, sub = (warp - 2) >> 2;
      const uint32_t stage = smem_u32(ctrl) + 1024u;
      SkCursor cur;
      sk_cursor_init(s, unit, cur);
      SkSeg seg;
      bool dead = false;
      while (sk_next(s, unit, cur, seg)) {
        const uint32_t buf = nseg & 1u;
        if (!dead) {
          const bool got = sk_wait_bar(tmem_full0 + 8u * buf, (nseg >> 1) & 1u, abort_flag, p, 24 + buf, 2);
          if (!__all_sync(0xffffffffu, got)) dead = true;
        }
        ++nseg;
        tc_fence_after();
        int tr, tc;
        sk_tile_mn(s, seg.tile, tr, tc);
        const int r0 = (tr * 2 + rank) * BM + q * 32, c0 = tc * p.bn;
        int valid_cols = p.cols - c0;
        if (valid_cols > p.bn) valid_cols = p.bn;
        const int blk = c0 / peer_set.block_cols;     // (tiles never straddle blocks: checked by the launcher)
        if (!dead && r0 < p.rows)
          sk_store_tile_tma_f32(&peer_set.tm[blk], stage, warp - 2, lane,
                                tmem_base + buf * BN + (static_cast<uint32_t>(q * 32) << 16), r0,
                                c0 - blk * peer_set.block_cols, valid_cols, sub, EPI_WARPS / 4);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(tmem_empty0 + 8u * buf);
      }
      if (lane == 0) tma_store_wait_read<0>();
    } else {
    sk_epilogue_loop<SK_EPI_ANY, EPI_WARPS>(p, C, unit, rank, warp, lane, tmem_base, tmem_full0, tmem_empty0,
                                            &ctrl->bcast, abort_flag, ctrl->pend, &tmC, cstage, &nseg, peers);
    }
    if (OUT != OUT_SCATTER && p.wide_units > 0) {
      // ---- wide units: the two halves are two whole tiles in the two accumulator buffers
      const int q = warp & 3;
      const int sub = (warp - 2) >> 2;   // the quadrant's two warps take alternate column groups
      const int row = q * 32 + lane;
      uint32_t groups = 0;
      bool dead = false;
      for (int u = unit; u < p.wide_units; u += s.grid) {
        int tm, tnw;
        sk_raster_mn(s, u, tm, tnw);
        const int r0 = (tm * 2 + rank) * BM;
        const bool row_ok = r0 + row < p.rows;
        const bool warp_ok = r0 + q * 32 < p.rows;
        for (int h = 0; h < 2; ++h, ++nseg) {
          const uint32_t buf = nseg & 1u;
          if (!dead) {
            const bool got = sk_wait_bar(tmem_full0 + 8u * buf, (nseg >> 1) & 1u, abort_flag, p, 24 + buf, 2);
            if (!__all_sync(0xffffffffu, got)) dead = true;
          }
          tc_fence_after();
          const int c0 = (2 * tnw + h) * BN;
          int valid_cols = p.cols - c0;
          if (valid_cols > BN) valid_cols = BN;
          const uint32_t t_addr = tmem_base + buf * BN + (static_cast<uint32_t>(q * 32) << 16);
          if (warp_ok && !dead && valid_cols > 0) {
            int c_first = 0;
            if (cstage != 0)
              c_first = sk_store_tile_tma<1>(p, &tmC, cstage, warp - 2, lane, t_addr, 0, r0 + q * 32, c0,
                                             valid_cols, groups, peers, sub, EPI_WARPS / 4) >> 5;
            for (int c = c_first + sub; c < ((valid_cols + 31) >> 5); c += EPI_WARPS / 4) {
              float v[32];
              sk_load_acc(t_addr + c * 32, 0, v);
              int nv = valid_cols - c * 32;
              if (nv > 32) nv = 32;
              if (row_ok) sk_store_chunk(C, p, r0 + row, c0 + c * 32, nv, v, peers);
            }
          }
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(tmem_empty0 + 8u * buf);
        }
      }
      if (cstage != 0 && lane == 0) tma_store_wait_read<0>();
    }
  }

  // ------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if constexpr (OUT != OUT_SCATTER) sk_reduce_pending(p, C, unit, rank, ctrl->pend, ctrl->ok, peers);
  // Neither CTA may leave while its partner can still signal its barriers or read its
  // shared memory.
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    if (*abort_flag) {
      const unsigned long long t0 = globaltimer_ns();
      while (globaltimer_ns() - t0 < 200000ULL) __nanosleep(1000);
    }
    tc_fence_after();
    __syncwarp();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
    if (lane == 0) sk_trace(p, 7);
  }
}

}  // namespace

int sk_make_tmap_f16(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols,
                     uint64_t ld_elems, uint32_t box_cols, uint32_t box_rows);

// fp32 row-major [rows, cols] tensor map with a 32 x 32 box (128-byte rows), 128-byte swizzle.
static int make_tmap_f32_store(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld) {
  typedef CUresult (*Fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                         const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                         CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static Fn enc = []() -> Fn {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess) return nullptr;
    return q == cudaDriverEntryPointSuccess ? reinterpret_cast<Fn>(f) : nullptr;
  }();
  if (!enc) return SK_ERR_LAUNCH;
  cuuint64_t gdim[2] = {cols, rows};
  cuuint64_t gstride[1] = {ld * 4};
  cuuint32_t box[2] = {32, 32};
  cuuint32_t estr[2] = {1, 1};
  const CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(base), gdim, gstride, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? SK_OK : sk_set_driver_error(static_cast<int>(r));
}

// Launch with CTA pairs.  `units` persistent pairs; p->sched must have been built for
// 256-row tiles and `units` schedulable units.  n_peers > 0: the fused all-gather; n_peers < 0:
// the fused reduce-scatter with -n_peers column blocks, peer_c[j] the fp32 receive slot of block j.
int sk_launch_f16_2cta(const sk_problem* prob, const void* A, const void* B, void* C, SkParams* p,
                       void* const* peer_c, int n_peers, void* stream) {
  const int n_blocks = n_peers < 0 ? -n_peers : 0;
  if (n_blocks) n_peers = 0;
  CUtensorMap tmA, tmB;
  int st = sk_make_tmap_f16(&tmA, A, prob->M, prob->K, prob->lda, BK, BM);
  if (st != SK_OK) return st;
  const int bn = p->bn;   // tile columns (sk_make_sched): 256, or narrower when asked for (multiple of 16)
  st = sk_make_tmap_f16(&tmB, B, prob->N, prob->K, prob->ldb, BK, bn / 2);
  CUtensorMap tmC;
  memset(&tmC, 0, sizeof(tmC));
  p->c_tma = p->c_vec_ok;   // whole tiles leave through shared memory and TMA stores
  if (n_blocks) p->c_tma = 0;
  if (st == SK_OK && p->c_tma) st = sk_make_tmap_f16(&tmC, C, prob->M, prob->N, prob->ldc, 64, 32);
  if (st != SK_OK) return st;
  SkPeers peer_set;
  memset(&peer_set, 0, sizeof(peer_set));
  if (n_blocks) {
    if (n_blocks > SK_MAX_TARGETS || !peer_c) return SK_ERR_ARG;
    if (prob->N % n_blocks != 0) return SK_ERR_SHAPE;
    const int bc = prob->N / n_blocks;
    // whole tiles only, none straddling two blocks; fp32 rows 16-byte aligned
    if (prob->schedule != SK_SCHED_DP || (bc % bn) != 0 || (bc & 3) != 0) return SK_ERR_SHAPE;
    peer_set.n = n_blocks;
    peer_set.block_cols = bc;
    for (int j = 0; j < n_blocks; ++j) {
      if (!peer_c[j]) return SK_ERR_ARG;
      if ((reinterpret_cast<uintptr_t>(peer_c[j]) & 15u) != 0) return SK_ERR_ALIGN;
      peer_set.c[j] = peer_c[j];
      st = make_tmap_f32_store(&peer_set.tm[j], peer_c[j], prob->M, bc, bc);
      if (st != SK_OK) return st;
    }
  }
  if (n_peers > 0) {
    if (n_peers > SK_MAX_PEERS || !peer_c) return SK_ERR_ARG;
    if (!p->c_vec_ok) return SK_ERR_ALIGN;
    peer_set.n = n_peers;
    for (int i = 0; i < n_peers; ++i) {
      if (!peer_c[i]) return SK_ERR_ARG;
      if ((reinterpret_cast<uintptr_t>(peer_c[i]) & 15u) != 0) return SK_ERR_ALIGN;
      peer_set.c[i] = peer_c[i];
      st = sk_make_tmap_f16(&peer_set.tm[i], peer_c[i], prob->M, prob->N, prob->ldc, 64, 32);
      if (st != SK_OK) return st;
    }
  }
  p->unit_ctas = 2;
  // Wide units (256 x 512, two column-adjacent tiles sharing every A stage): decided by the host
  // scheduler (sk_make_sched), which leaves their count in wide_base.
  p->wide_units = p->sched.wide_base > 0 ? p->sched.wide_base : 0;
  p->acc_stride = BN;           // (the accumulator buffers stay 256 columns apart)
  p->col_tx_bytes = (bn / 2) * BK * 2;   // bytes of this CTA's half of a B stage
  p->tmem_cols = TMEM_COLS;
  p->stages = STAGES;
  p->idesc = umma_idesc_f16(2 * BM, bn, 0, p->out_bf16);
  // K steps the second half of a 256 x 512 unit stays behind the first (see the MMA issuer).
  // Measured on configuration 5, sustained loop: 1278 TFLOP/s with 0, 1291 with 1, 1137 with 2
  // (two held stages leave the producer too little room).
  p->wide_lag = 1;

  static SkPerDeviceOnce attrs;
  cudaError_t e = attrs.run([]() {
    cudaError_t r = cudaFuncSetAttribute(sk_gemm_f16_2cta_kernel<OUT_PLAIN>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (r == cudaSuccess)
      r = cudaFuncSetAttribute(sk_gemm_f16_2cta_kernel<OUT_GATHER>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               SMEM_BYTES);
    if (r == cudaSuccess)
      r = cudaFuncSetAttribute(sk_gemm_f16_2cta_kernel<OUT_SCATTER>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               SMEM_BYTES);
    return r;
  });
  if (e != cudaSuccess) return sk_set_cuda_error(e);
  const bool pdl = (prob->flags & SK_FLAG_PDL) != 0;
  const cudaStream_t cs = static_cast<cudaStream_t>(stream);
  __half* Ch = static_cast<__half*>(C);
  if (n_blocks)
    e = sk_launch(sk_gemm_f16_2cta_kernel<OUT_SCATTER>, p->sched.grid * 2, NUM_THREADS, SMEM_BYTES, cs, 2, pdl,
                  tmA, tmB, tmC, Ch, *p, peer_set);
  else if (n_peers > 0)
    e = sk_launch(sk_gemm_f16_2cta_kernel<OUT_GATHER>, p->sched.grid * 2, NUM_THREADS, SMEM_BYTES, cs, 2, pdl,
                  tmA, tmB, tmC, Ch, *p, peer_set);
  else
    e = sk_launch(sk_gemm_f16_2cta_kernel<OUT_PLAIN>, p->sched.grid * 2, NUM_THREADS, SMEM_BYTES, cs, 2, pdl,
                  tmA, tmB, tmC, Ch, *p, peer_set);
  if (e != cudaSuccess) return sk_set_cuda_error(e);
  return SK_OK;
}
