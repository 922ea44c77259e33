// W4A16 Stream-K GEMM on sm_100a: C[M,N] = A[M,K] . W^T, W = (q - z) * s with
// uint4 q, per-group (128 along K) uint4 zero-point z and fp16 scale s.
//
// Stands in for the TL kernel of streamk_fp16_ladder_block_reduce_q4.py:143-522
// (int8-packed weight tile in shared memory, decode_i4u_to_f16 in registers, then
// mma.sync) and for its CPU weight preparation (LadderPermutate + LOP3Permutate,
// …q4.py:568-595).  The reference applies no scale or zero-point; with s = 1,
// z = 0 this kernel computes the same C = A . unpack_u4(qB)^T.
//
// Packed image (sk_prepack_q4):
//   nibble blocks  [n_block][k_block] of 128 rows x 64 K = 4096 B, stored as
//                  [half h][row r][16 B]; the 16 B hold K = h*32 .. h*32+31 of row r
//                  as four words, each word's eight nibbles in the order
//                  e0 e2 e4 e6 e1 e3 e5 e7 so that (w >> 4i) & 0x000F000F yields
//                  the fp16 pair (e(2i), e(2i+1)) in one lop3;
//   group blocks   [n_block][group] = 128 fp16 scales + 128 uint8 zero-points (384 B).
//
// CTA roles (448 threads): warp 0 producer (TMA activation tile + bulk copies of the
// packed blocks), warp 1 MMA issuer, warps 2..5 epilogue, warps 6..13 dequantise the
// packed block into the 128-byte-swizzled fp16 stage the UMMA descriptor reads.  For short
// M the operands are swapped: the dequantised weights feed the UMMA M dimension and the
// activation tile (M rounded up to 16 rows) the N dimension.
#include "sk_common.cuh"
#include "sk_epilogue.cuh"

namespace {

using namespace skptx;

constexpr int BM = SK_BM;
constexpr int BK = 64;
constexpr int Q_BLOCK_BYTES = 128 * BK / 2;    // 4096: packed nibbles of 128 weight rows x 64 K
constexpr int SZ_BLOCK_BYTES = 128 * 2 + 128;  // 384: fp16 scales + uint8 zero-points of a group
constexpr int W_SLAB_BYTES = 128 * BK * 2;     // 16384: dequantised fp16 tile of one K step
constexpr int KG = 2;                          // K steps per stage = one scale group (128 along K)
constexpr int W_STAGE_BYTES = KG * W_SLAB_BYTES;
constexpr int MAX_LS = 12;                     // load stages (activation tile + packed block)
constexpr int MAX_BS = 8;                      // dequantised weight stages (ring depth chosen per launch)
constexpr int DQ_WARPS = 8;
constexpr int DQ_GROUPS = 4;                   // groups of DQ_WARPS / DQ_GROUPS warps, one stage each at a time
constexpr int DQ_GROUP_WARPS = DQ_WARPS / DQ_GROUPS;
constexpr int DQ_THREADS = DQ_WARPS * 32;
constexpr int NUM_THREADS = 64 + SK_EPI_THREADS + DQ_THREADS + 32;   // + warp 14, the second MMA issuer
constexpr int MMA_B_WARP = 6 + DQ_WARPS;
constexpr int CTRL_BYTES = 512;
constexpr int SMEM_LIMIT = 232448;

struct Ctrl {
  uint64_t load_full[MAX_LS];
  uint64_t load_empty[MAX_LS];
  uint64_t w_full[MAX_BS];
  uint64_t w_empty[MAX_BS];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint64_t recv_full;      // SK_SCHED_CLUSTER: the partial tiles of the other CTAs have arrived
  uint32_t tmem_base;
  uint32_t abort;
  uint32_t bcast;
  uint32_t ok[2];
  SkPending pend[2];
};
static_assert(sizeof(Ctrl) <= CTRL_BYTES, "Ctrl must fit its reserved space");

// Eight uint4 values of one packed word -> eight fp16 (q - z) * s, in K order.
// zmagic = half2(1024 + z), s2 = half2(s, s).  The subtraction is exact and the
// product is rounded once, exactly like ((q.half() - z.half()) * s) on the CPU.
__device__ __forceinline__ uint4 dequant_word(uint32_t w, __half2 zmagic, __half2 s2) {
  constexpr uint32_t MASK = 0x000F000Fu;
  constexpr uint32_t MAGIC = 0x64006400u;  // fp16 1024.0 in both halves
  uint32_t t[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t sh = w >> (4 * i);
    // (sh & MASK) | MAGIC in one lop3 (truth table 0xEA = (a & b) | c)
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(t[i]) : "r"(sh), "r"(MASK), "r"(MAGIC));
  }
  uint32_t o[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __half2 x = *reinterpret_cast<const __half2*>(&t[i]);
    const __half2 y = __hmul2(__hsub2(x, zmagic), s2);
    o[i] = *reinterpret_cast<const uint32_t*>(&y);
  }
  return make_uint4(o[0], o[1], o[2], o[3]);
}

// Shared memory: [BS dequantised weight stages][LS activation stages][LS packed blocks]
// [LS group blocks][Ctrl]; BS and LS are chosen per launch.  p.col_stage_bytes holds the activation stage size in both
// operand orders (128 rows normally, bn rows when the operands are swapped).
// MODE as in the fp16 kernel: SK_EPI_ATOMIC, SK_EPI_BLOCK_REDUCE, SK_EPI_WHOLE (data-parallel
// schedule, no fixup code) or SK_MODE_CLUSTER; one instantiation each.
constexpr int SK_MODE_CLUSTER = 3;

template <int MODE>
__global__ void __launch_bounds__(NUM_THREADS, 1)
sk_gemm_w4a16_kernel(const __grid_constant__ CUtensorMap tmA, const uint8_t* __restrict__ qblocks,
                     const uint8_t* __restrict__ szblocks, __half* __restrict__ C, const SkParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw_addr);
  const int LS = p.stages;
  const int BS = p.w_stages;
  const int a_tile_bytes = p.row_tx_bytes;         // activation tile bytes of one K step
  const int a_stage_bytes = KG * a_tile_bytes;
  const int off_a = BS * W_STAGE_BYTES;
  const int off_q = off_a + LS * a_stage_bytes;
  const int off_sz = off_q + LS * KG * Q_BLOCK_BYTES;
  const uint32_t sW = base;
  const uint32_t sA = base + off_a;
  const uint32_t sQ = base + off_q;
  const uint32_t sSZ = base + off_sz;
  Ctrl* ctrl = reinterpret_cast<Ctrl*>(smem + off_sz + LS * SZ_BLOCK_BYTES);
  volatile uint32_t* abort_flag = &ctrl->abort;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int pid = blockIdx.x;
  const SkSched& s = p.sched;
  const int kblocks = s.iters_per_tile;  // K / 64
  const int groups = kblocks >> 1;       // K / 128
  const bool swapped = p.transposed != 0;
  if (threadIdx.x == 0) {
    sk_trace(p, 0);
    griddep_launch_dependents();   // the next kernel of the stream may begin its own start-up
  }
  // Split-K inside a cluster (sk_epilogue.cuh): receive buffer behind the control block,
  // staging area in the rings, which are idle by then.
  constexpr bool clustered = MODE == SK_MODE_CLUSTER;
  const uint32_t recv_base = smem_u32(ctrl) + CTRL_BYTES;

  if (threadIdx.x == 0) {
    if (clustered) mbar_init(smem_u32(&ctrl->recv_full), 5);   // 4 epilogue warps + the byte count
    for (int i = 0; i < LS; ++i) {
      mbar_init(smem_u32(&ctrl->load_full[i]), 1);
      mbar_init(smem_u32(&ctrl->load_empty[i]), DQ_GROUP_WARPS + 1);  // the stage's dequant warps + MMA commit
    }
    for (int i = 0; i < BS; ++i) {
      mbar_init(smem_u32(&ctrl->w_full[i]), DQ_GROUP_WARPS);   // one arrival per dequant warp of the stage's group
      mbar_init(smem_u32(&ctrl->w_empty[i]), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&ctrl->tmem_full[i]), p.acc_b_off ? 2 : 1);   // one arrival per MMA issuer
      mbar_init(smem_u32(&ctrl->tmem_empty[i]), 4);
    }
    ctrl->abort = 0u;
    ctrl->bcast = 0u;
    ctrl->pend[0].tile = -1;
    ctrl->pend[1].tile = -1;
    fence_mbar_init();
    fence_proxy_async_smem();
    prefetch_tensormap(&tmA);
    if (clustered)
      mbar_arrive_expect_tx(smem_u32(&ctrl->recv_full),
                            static_cast<uint32_t>((s.split - 1) * p.cl_per) * SK_CL_QUAD_BYTES);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&ctrl->tmem_base), p.tmem_cols);
    tmem_relinquish();
  }
  if (threadIdx.x == 64) {
    // While the barriers are being set up (and, with SK_FLAG_PDL, while the previous kernel of
    // the stream is still running) an idle thread asks L2 for the packed weights of the first
    // stages (a hint; L2 is the coherence point, so nothing can go stale).
    SkCursor c0;
    sk_cursor_init(s, pid, c0);
    SkSeg g0;
    if (sk_next(s, pid, c0, g0)) {
      int tr, tc;
      sk_tile_mn(s, g0.tile, tr, tc);
      const int nblk = swapped ? tr : tc;
      int n = g0.k1 - g0.k0;
      if (n > 8) n = 8;
      bulk_prefetch_l2(qblocks + (static_cast<size_t>(nblk) * kblocks + g0.k0) * Q_BLOCK_BYTES,
                       static_cast<uint32_t>(n) * Q_BLOCK_BYTES);
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&ctrl->tmem_base);
  if (threadIdx.x == 0) sk_trace(p, 1);
  // global memory is the previous kernel's until it has completed (no-op without SK_FLAG_PDL)
  griddep_wait();

  if (warp == 0) {
    // ------------------------------------------------------------- producer
    if (lane == 0) {
      bool traced = false;
      bool arrived = false;   // this thread's share of the cluster's start-up barrier
      SkCursor cur;
      sk_cursor_init(s, pid, cur);
      SkSeg seg;
      int ls = 0;
      uint32_t lph = 0;
      bool ok = true;
      while (ok && sk_next(s, pid, cur, seg)) {
        int tr, tc;
        sk_tile_mn(s, seg.tile, tr, tc);
        const int nblk = swapped ? tr : tc;                  // 128-row block of the weight
        const int a_row0 = swapped ? tc * p.bn : tr * BM;    // first activation row of the tile
        for (int k = seg.k0; k < seg.k1;) {
          // A stage carries the K steps of one scale group (two, unless the segment starts
          // or ends inside the group): one barrier round trip, one packed copy, one group block.
          const int n = ((k & 1) || k + 1 >= seg.k1) ? 1 : 2;
          const uint32_t full = smem_u32(&ctrl->load_full[ls]);
          if (!sk_wait_bar(smem_u32(&ctrl->load_empty[ls]), lph ^ 1u, abort_flag, p, ls, 0)) {
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(full, n * (a_tile_bytes + Q_BLOCK_BYTES) + SZ_BLOCK_BYTES);
          for (int j = 0; j < n; ++j)
            tma_load_2d(sA + ls * a_stage_bytes + j * a_tile_bytes, &tmA, full, (k + j) * BK, a_row0);
          bulk_load_1d(sQ + ls * KG * Q_BLOCK_BYTES,
                       qblocks + (static_cast<size_t>(nblk) * kblocks + k) * Q_BLOCK_BYTES,
                       n * Q_BLOCK_BYTES, full);
          bulk_load_1d(sSZ + ls * SZ_BLOCK_BYTES,
                       szblocks + (static_cast<size_t>(nblk) * groups + (k >> 1)) * SZ_BLOCK_BYTES,
                       SZ_BLOCK_BYTES, full);
          k += n;
          if (++ls == LS) {
            ls = 0; lph ^= 1u;
            // ring full for the first time; this thread initialised the mbarriers the other
            // CTAs will signal, so its arrival releases
            if (clustered && !arrived) { cluster_arrive(); arrived = true; }
          }
          if (!traced) { sk_trace(p, 2); traced = true; }
        }
      }
      if (clustered && !arrived) cluster_arrive();
    } else if (clustered) {
      cluster_arrive_relaxed();
    }
  } else if (warp == 1 || warp == MMA_B_WARP) {
    // ------------------------------------------------------------- MMA issuers
    // Issuing a UMMA costs its thread about 50 ns, and with eight per stage this thread was
    // the mainloop's limit.  With room in tensor memory for two accumulators per buffer
    // (p.acc_b_off), a second thread takes every other stage of a segment and accumulates on
    // its own; the epilogue adds the two.
    const uint32_t me = warp == 1 ? 0u : 1u;
    if (lane == 0 && (me == 0u || p.acc_b_off != 0)) {
      const bool dual = p.acc_b_off != 0;
      SkCursor cur;
      sk_cursor_init(s, pid, cur);
      SkSeg seg;
      int ls = 0, bs = 0;
      uint32_t lph = 0, bph = 0, nseg = 0;
      bool ok = true;
      bool arrived = false;
      const uint64_t desc_hi = umma_desc_sw128_hi(16, 1024);
      const uint32_t act_lo0 = umma_desc_lo(sA), wgt_lo0 = umma_desc_lo(sW);
      const uint32_t act_tile16 = static_cast<uint32_t>(a_tile_bytes) >> 4;
      const uint32_t idesc = p.idesc;
      while (ok && sk_next(s, pid, cur, seg)) {
        const uint32_t buf = nseg & 1u;
        const uint32_t acc_ph = (nseg >> 1) & 1u;
        if (!sk_wait_bar(smem_u32(&ctrl->tmem_empty[buf]), acc_ph ^ 1u, abort_flag, p, 16 + buf, 1))
          break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * p.acc_stride + me * p.acc_b_off;
        uint32_t accumulate = 0u;   // this thread's first UMMA of the segment overwrites its accumulator
        uint32_t si = 0;            // stage number inside the segment
        for (int k = seg.k0; k < seg.k1; ++si) {
          const int n = ((k & 1) || k + 1 >= seg.k1) ? 1 : 2;
          // (both issuers watch every stage's barriers complete, in order: see the dequant warps)
          if (!sk_wait_bar(smem_u32(&ctrl->load_full[ls]), lph, abort_flag, p, 32 + ls, 1) ||
              !sk_wait_bar(smem_u32(&ctrl->w_full[bs]), bph, abort_flag, p, 48 + bs, 1)) {
            ok = false;
            break;
          }
          if (!dual || (si & 1u) == me) {
            tc_fence_after();
            if (nseg == 0 && k == seg.k0) sk_trace(p, 3);
            for (int j = 0; j < n; ++j) {
              const uint32_t act = act_lo0 + (ls * KG + j) * act_tile16;
              const uint32_t wgt = wgt_lo0 + (bs * KG + j) * (W_SLAB_BYTES >> 4);
              const uint32_t a_lo = swapped ? wgt : act;   // UMMA M side
              const uint32_t b_lo = swapped ? act : wgt;   // UMMA N side
#pragma unroll
              for (int kk = 0; kk < BK / 16; ++kk) {
                umma_f16_ss(d_tmem, desc_hi | (a_lo + kk * 2), desc_hi | (b_lo + kk * 2), idesc, accumulate);
                accumulate = 1u;
              }
            }
            umma_commit(smem_u32(&ctrl->load_empty[ls]));
            umma_commit(smem_u32(&ctrl->w_empty[bs]));
            if (clustered && !arrived) { cluster_arrive_relaxed(); arrived = true; }
          }
          k += n;
          if (++ls == LS) { ls = 0; lph ^= 1u; }
          if (++bs == BS) { bs = 0; bph ^= 1u; }
        }
        if (!ok) break;
        // (a thread that issued nothing in this segment has nothing to wait for)
        if (accumulate) umma_commit(smem_u32(&ctrl->tmem_full[buf]));
        else mbar_arrive(smem_u32(&ctrl->tmem_full[buf]));
        ++nseg;
      }
      if (me == 0u) sk_trace(p, 4);
      if (clustered && !arrived) cluster_arrive_relaxed();
    } else if (clustered) {
      cluster_arrive_relaxed();
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------- epilogue
    if constexpr (clustered)   // (takes part in the cluster's start-up barrier on its own)
      sk_cluster_send(p, static_cast<int>(cluster_ctarank()), warp, lane, tmem_base,
                      smem_u32(&ctrl->tmem_full[0]), sW, recv_base, smem_u32(&ctrl->recv_full),
                      abort_flag, sk_cta_begin(s, pid) % s.iters_per_tile,
                      sk_cta_begin(s, pid + 1) - sk_cta_begin(s, pid));
    else
      sk_epilogue_loop<MODE>(p, C, pid, 0, warp, lane, tmem_base, smem_u32(&ctrl->tmem_full[0]),
                             smem_u32(&ctrl->tmem_empty[0]), &ctrl->bcast, abort_flag, ctrl->pend);
  } else {
    // ------------------------------------------------------------- dequantise
    // The eight warps form four groups of two, and group g takes stages g, g+4, g+8, ... whole.
    // A stage costs a group far more in fixed latencies (two barrier waits, the loads of the
    // packed words, scales and zero-points, the proxy fence, the arrivals) than in arithmetic,
    // so what counts is how many stages are in flight at once, not how many threads share one:
    // with every warp working on every stage, as a first version did, the stage rate was one
    // warp's latency chain (0.8 us per stage, whatever was removed from it).
    // Thread t of a group handles the 16-byte units u = t, t+64, t+128, t+192 of a K step:
    // unit u = weight row u & 127, K half u >> 7 (32 values = 4 packed words).
    const int dw = warp - 6;
    const int grp = dw >> 1;
    const int t = (dw & 1) * 32 + lane;
    SkCursor cur;
    sk_cursor_init(s, pid, cur);
    SkSeg seg;
    int ls = 0, bs = 0;
    uint32_t lph = 0, bph = 0;
    uint32_t sidx = 0;   // running stage number
    bool dead = false;
    if (clustered) cluster_arrive_relaxed();
    while (sk_next(s, pid, cur, seg)) {
      for (int k = seg.k0; k < seg.k1;) {
        const int n = ((k & 1) || k + 1 >= seg.k1) ? 1 : 2;
        // Every warp watches every stage's barriers complete, in order, also those of the
        // stages it does not work on: a parity wait only tells a phase from its neighbours, and
        // a group that skipped phases could take a slot's previous use for the awaited one
        // (its stages are four apart, the rings may be shorter).  Both barriers of a foreign
        // stage complete before those of the group's own next stage, so this costs no time.
        if (!dead) {
          if (!sk_wait_bar(smem_u32(&ctrl->load_full[ls]), lph, abort_flag, p, 64 + ls, 3) ||
              !sk_wait_bar(smem_u32(&ctrl->w_empty[bs]), bph ^ 1u, abort_flag, p, 80 + bs, 3))
            dead = true;
        }
        if ((sidx & (DQ_GROUPS - 1)) == static_cast<uint32_t>(grp)) {
          if (!dead) {
            const uint8_t* sz = smem + off_sz + ls * SZ_BLOCK_BYTES;
            // rows t and t + 64
            __half2 s2[2], zmagic[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const int r = t + 64 * e;
              const __half sc = *reinterpret_cast<const __half*>(sz + r * 2);
              const uint32_t z = sz[256 + r];
              s2[e] = __half2half2(sc);
              const uint32_t zm = 0x64006400u | z | (z << 16);
              zmagic[e] = *reinterpret_cast<const __half2*>(&zm);
            }
            for (int j = 0; j < n; ++j) {
              const uint8_t* q = smem + off_q + (ls * KG + j) * Q_BLOCK_BYTES;
              uint8_t* slab = smem + (bs * KG + j) * W_SLAB_BYTES;
              uint4 w[4];
#pragma unroll
              for (int i = 0; i < 4; ++i) w[i] = *reinterpret_cast<const uint4*>(q + (t + 64 * i) * 16);
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const int u = t + 64 * i;
                const int r = u & 127, h = u >> 7, e = i & 1;
                uint8_t* wrow = slab + r * 128;
                const int sw = r & 7;
                const uint32_t words[4] = {w[i].x, w[i].y, w[i].z, w[i].w};
#pragma unroll
                for (int c = 0; c < 4; ++c)
                  *reinterpret_cast<uint4*>(wrow + (((h * 4 + c) ^ sw) << 4)) =
                      dequant_word(words[c], zmagic[e], s2[e]);
              }
            }
            fence_proxy_async_smem();  // generic-proxy stores -> visible to the UMMA reads
          }
          __syncwarp();
          if (lane == 0) {
            mbar_arrive(smem_u32(&ctrl->w_full[bs]));
            mbar_arrive(smem_u32(&ctrl->load_empty[ls]));
          }
        }
        ++sidx;
        k += n;
        if (++ls == LS) { ls = 0; lph ^= 1u; }
        if (++bs == BS) { bs = 0; bph ^= 1u; }
      }
    }
  }

  // ------------------------------------------------------------- teardown
  tc_fence_before();
  bool reduce_ok = true;
  if constexpr (clustered) {
    if (!(warp >= 2 && warp < 6)) cluster_wait();   // start-up barrier, second half
    __syncwarp();
    // the chunks of the other CTAs, and the epilogue warps' own one
    reduce_ok = sk_wait_bar(smem_u32(&ctrl->recv_full), 0u, abort_flag, p, 40, 3);
    // Final barrier: nobody leaves while a copy out of its staging area may be in flight.
    // Arrive now, wait after the reduction.
    cluster_arrive();
    if (threadIdx.x == 0) sk_trace(p, 6);
  } else {
    __syncthreads();
  }
  // The accumulators have been read: the tensor memory can go back while the rest reduces.
  if (warp == 1) {
    if (*abort_flag) {
      const unsigned long long t0 = globaltimer_ns();
      while (globaltimer_ns() - t0 < 200000ULL) __nanosleep(1000);
    }
    tc_fence_after();
    __syncwarp();
    tmem_dealloc(tmem_base, p.tmem_cols);
  }
  if constexpr (clustered) {
    if (reduce_ok)
      sk_cluster_reduce(p, C, pid >> s.split_log2, static_cast<int>(cluster_ctarank()), recv_base);
    cluster_wait();
  } else {
    // Block-reduce fixup: every thread of the CTA now helps to reduce this CTA's slices of
    // the split tiles it took part in.
    if constexpr (MODE == SK_EPI_BLOCK_REDUCE) sk_reduce_pending(p, C, pid, 0, ctrl->pend, ctrl->ok);
  }
  if (threadIdx.x == 32) sk_trace(p, 7);
}

// ---------------------------------------------------------------- prepack / dequant
// One thread per output word.  Source nibble e of an 8-element group sits at bits 4e.
__global__ void prepack_q4_kernel(const uint32_t* __restrict__ qw, const __half* __restrict__ scales,
                                  const uint8_t* __restrict__ zeros, int N, int K,
                                  uint32_t* __restrict__ qout, uint8_t* __restrict__ szout,
                                  int nblocks, int kblocks) {
  const int kwords = K / 8;
  const int groups = K / 128;
  const size_t total_words = static_cast<size_t>(nblocks) * kblocks * 1024;
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total_words;
       i += stride) {
    const size_t blk = i >> 10;
    const int in_blk = static_cast<int>(i & 1023);
    const int h = in_blk >> 9;
    const int r = (in_blk >> 2) & 127;
    const int j = in_blk & 3;
    const int nb = static_cast<int>(blk / kblocks);
    const int kb = static_cast<int>(blk - static_cast<size_t>(nb) * kblocks);
    const int n = nb * 128 + r;
    uint32_t out = 0u;
    if (n < N) {
      const uint32_t w = qw[static_cast<size_t>(n) * kwords + kb * 8 + h * 4 + j];
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        out |= ((w >> (8 * t)) & 0xFu) << (4 * t);            // even elements 0,2,4,6
        out |= ((w >> (8 * t + 4)) & 0xFu) << (4 * (t + 4));  // odd elements 1,3,5,7
      }
    }
    qout[i] = out;
  }
  const size_t total_sz = static_cast<size_t>(nblocks) * groups * 128;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total_sz;
       i += stride) {
    const size_t gblk = i >> 7;
    const int r = static_cast<int>(i & 127);
    const int nb = static_cast<int>(gblk / groups);
    const int g = static_cast<int>(gblk - static_cast<size_t>(nb) * groups);
    const int n = nb * 128 + r;
    __half sc = __float2half(0.f);
    uint8_t z = 0;
    if (n < N) {
      sc = scales ? scales[static_cast<size_t>(n) * groups + g] : __float2half(1.f);
      z = zeros ? static_cast<uint8_t>(zeros[static_cast<size_t>(n) * groups + g] & 0xF) : 0;
    }
    uint8_t* dst = szout + gblk * SZ_BLOCK_BYTES;
    *reinterpret_cast<__half*>(dst + r * 2) = sc;
    dst[256 + r] = z;
  }
}

// One thread per packed word -> eight halves of W[n, k..k+7].
__global__ void dequant_q4_kernel(const uint32_t* __restrict__ qblocks,
                                  const uint8_t* __restrict__ szblocks, int N, int K,
                                  __half* __restrict__ W, int ldw, int kblocks) {
  const int groups = K / 128;
  const size_t nb_used = (static_cast<size_t>(N) + 127) / 128;
  const size_t total_words = nb_used * kblocks * 1024;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total_words;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t blk = i >> 10;
    const int in_blk = static_cast<int>(i & 1023);
    const int h = in_blk >> 9;
    const int r = (in_blk >> 2) & 127;
    const int j = in_blk & 3;
    const int nb = static_cast<int>(blk / kblocks);
    const int kb = static_cast<int>(blk - static_cast<size_t>(nb) * kblocks);
    const int n = nb * 128 + r;
    if (n >= N) continue;
    const uint8_t* sz = szblocks + (static_cast<size_t>(nb) * groups + (kb >> 1)) * SZ_BLOCK_BYTES;
    const __half sc = *reinterpret_cast<const __half*>(sz + r * 2);
    const uint32_t z = sz[256 + r];
    const uint32_t zm = 0x64006400u | z | (z << 16);
    const uint4 o = dequant_word(qblocks[i], *reinterpret_cast<const __half2*>(&zm), __half2half2(sc));
    __half* dst = W + static_cast<size_t>(n) * ldw + kb * 64 + h * 32 + j * 8;
    if ((reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
      *reinterpret_cast<uint4*>(dst) = o;
    } else {
      const __half* hv = reinterpret_cast<const __half*>(&o);
#pragma unroll
      for (int e = 0; e < 8; ++e) dst[e] = hv[e];
    }
  }
}

inline int q4_nblocks(int N) { return (N + 255) / 256 * 2; }

}  // namespace

int sk_make_tmap_f16(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols,
                     uint64_t ld_elems, uint32_t box_cols, uint32_t box_rows);
void sk_fill_tile_params(SkParams* p, int bn, int stage_fixed_bytes, int max_stages,
                         int reserved_bytes, bool two_issuers);

extern "C" size_t sk_q4_bytes(int N, int K) {
  if (N <= 0 || K <= 0 || (K % 128) != 0) return 0;
  const size_t nb = q4_nblocks(N);
  return nb * (K / 64) * Q_BLOCK_BYTES + nb * (K / 128) * SZ_BLOCK_BYTES;
}

extern "C" int sk_prepack_q4(const void* qweight, const void* scales, const void* zeros, int N,
                             int K, void* out, size_t out_bytes, void* stream) {
  if (!qweight || !out) return SK_ERR_ARG;
  if (N <= 0 || K <= 0 || (K % 128) != 0) return SK_ERR_SHAPE;
  if (out_bytes < sk_q4_bytes(N, K)) return SK_ERR_WORKSPACE;
  if ((reinterpret_cast<uintptr_t>(out) & 15u) || (reinterpret_cast<uintptr_t>(qweight) & 3u))
    return SK_ERR_ALIGN;
  const int nb = q4_nblocks(N), kb = K / 64;
  uint8_t* o = static_cast<uint8_t*>(out);
  uint8_t* sz = o + static_cast<size_t>(nb) * kb * Q_BLOCK_BYTES;
  const size_t total = static_cast<size_t>(nb) * kb * 1024;
  const int grid = static_cast<int>((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  prepack_q4_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint32_t*>(qweight), static_cast<const __half*>(scales),
      static_cast<const uint8_t*>(zeros), N, K, reinterpret_cast<uint32_t*>(o), sz, nb, kb);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return sk_set_cuda_error(e);
  return SK_OK;
}

extern "C" int sk_dequant_q4(const void* packed, int N, int K, void* W, int ldw, void* stream) {
  if (!packed || !W) return SK_ERR_ARG;
  if (N <= 0 || K <= 0 || (K % 128) != 0 || ldw < K) return SK_ERR_SHAPE;
  if (reinterpret_cast<uintptr_t>(packed) & 15u) return SK_ERR_ALIGN;
  const int nb = q4_nblocks(N), kb = K / 64;
  const uint8_t* o = static_cast<const uint8_t*>(packed);
  const uint8_t* sz = o + static_cast<size_t>(nb) * kb * Q_BLOCK_BYTES;
  const size_t total = (static_cast<size_t>(N) + 127) / 128 * kb * 1024;
  const int grid = static_cast<int>((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  dequant_q4_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const uint32_t*>(o), sz, N, K, static_cast<__half*>(W), ldw, kb);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return sk_set_cuda_error(e);
  return SK_OK;
}

extern "C" int sk_gemm_w4a16(const sk_problem* prob, const void* A, const void* packed, void* C,
                             void* ws, size_t ws_bytes, void* stream) {
  if (!prob || !A || !packed || !C) return SK_ERR_ARG;
  if (prob->fixup != SK_FIXUP_ATOMIC && prob->fixup != SK_FIXUP_BLOCK_REDUCE) return SK_ERR_ARG;
  int num_sms = 0, dev_sms = 0;
  int st = sk_resolve_grid(prob, &num_sms, &dev_sms);
  if (st != SK_OK) return st;
  sk_problem resolved = *prob;   // SK_SCHED_AUTO -> a concrete schedule and tile
  sk_resolve_auto(&resolved, 2, num_sms);
  prob = &resolved;
  const int M = prob->M, N = prob->N, K = prob->K;
  if (M <= 0 || N <= 0 || K <= 0 || (K % 128) != 0) return SK_ERR_SHAPE;
  if (prob->lda < K || prob->ldc < N) return SK_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(A) & 15u) || (reinterpret_cast<uintptr_t>(packed) & 15u))
    return SK_ERR_ALIGN;
  if ((prob->lda & 7) != 0 || (reinterpret_cast<uintptr_t>(C) & 1u) != 0) return SK_ERR_ALIGN;
  if (!ws || ws_bytes < sk_ws_total_bytes(dev_sms)) return SK_ERR_WORKSPACE;
  if ((reinterpret_cast<uintptr_t>(ws) & 255u) != 0) return SK_ERR_ALIGN;

  SkParams p;
  memset(&p, 0, sizeof(p));
  SkPlan plan;
  st = sk_make_sched(prob, 2, num_sms, nullptr, &p.sched, &plan);
  if (st != SK_OK) return st;
  p.M = M; p.N = N; p.K = K;
  p.lda = prob->lda; p.ldb = 0; p.ldc = prob->ldc;
  p.rows = plan.rows; p.cols = plan.cols;
  p.transposed = plan.swap;
  p.unit_ctas = 1;
  p.bm = BM;
  p.fixup = prob->fixup;
  p.c_vec_ok = ((reinterpret_cast<uintptr_t>(C) & 15u) == 0 && (prob->ldc & 7) == 0) ? 1 : 0;
  p.drop_flag_cta = prob->test_drop_flag_cta - 1;
  p.timeout_ns = (prob->fixup_timeout_us > 0 ? static_cast<unsigned long long>(prob->fixup_timeout_us)
                                             : 2000000ULL) * 1000ULL;
  p.ws = sk_ws_carve(ws, dev_sms);
  p.trace = sk_trace_buffer();
  // The activation tile has 128 rows normally, bn rows when the operands are swapped.
  const int a_rows = plan.swap ? plan.bn : BM;
  const int a_stage_bytes = a_rows * BK * 2;
  // (two MMA issuers pay off for the narrow UMMAs of the swapped order only: measured)
  sk_fill_tile_params(&p, plan.bn, 0, 1, 0, plan.swap != 0);   // TMEM layout only; stages set below
  p.kpair = 1;
  // Two rings share the shared memory: load stages (activation tile + packed block) and
  // dequantised weight stages.  The chain dequantise -> MMA -> release runs once per K step
  // and takes over a microsecond end to end, so the weight ring has to be deep as well: take
  // the deepest weight ring that still leaves at least as many load stages.
  const int split = p.sched.split;   // SK_SCHED_CLUSTER: CTAs per tile
  const int recv_bytes = split ? sk_cluster_recv_bytes(plan.bn, split) : 0;
  p.cl_per = split ? sk_cluster_quads_per_cta(plan.bn, split) : 1;
  p.cl_per_div = sk_div_make(p.cl_per);
  const int budget = SMEM_LIMIT - 1024 - CTRL_BYTES - recv_bytes;
  const int load_stage = KG * (a_stage_bytes + Q_BLOCK_BYTES) + SZ_BLOCK_BYTES;
  int ls = 0, bs = 2;
  for (int b = 4; b >= 2; --b) {
    const int l = (budget - b * W_STAGE_BYTES) / load_stage;
    if (l >= b || b == 2) { bs = b; ls = l; break; }
  }
  if (ls > 8) ls = 8;
  if (ls < 2) return SK_ERR_SHAPE;
  p.stages = ls;
  p.w_stages = bs;
  p.row_tx_bytes = a_stage_bytes;
  p.col_stage_bytes = a_stage_bytes;
  p.idesc = umma_idesc_f16(BM, plan.bn, 0);

  CUtensorMap tmA;
  st = sk_make_tmap_f16(&tmA, A, M, K, prob->lda, BK, a_rows);
  if (st != SK_OK) return st;
  const int nb = q4_nblocks(N), kb = K / 64;
  const uint8_t* qb = static_cast<const uint8_t*>(packed);
  const uint8_t* sz = qb + static_cast<size_t>(nb) * kb * Q_BLOCK_BYTES;

  // the staging area of the cluster exchange lives in the rings
  if (split && bs * W_STAGE_BYTES + ls * load_stage < recv_bytes) return SK_ERR_SHAPE;
  const int smem_bytes = bs * W_STAGE_BYTES + ls * load_stage + 1024 + CTRL_BYTES + recv_bytes;
  static SkPerDeviceOnce attrs;
  cudaError_t e = attrs.run([]() {
    cudaError_t r = cudaSuccess;
    const void* kernels[4] = {
        reinterpret_cast<const void*>(sk_gemm_w4a16_kernel<SK_EPI_ATOMIC>),
        reinterpret_cast<const void*>(sk_gemm_w4a16_kernel<SK_EPI_BLOCK_REDUCE>),
        reinterpret_cast<const void*>(sk_gemm_w4a16_kernel<SK_EPI_WHOLE>),
        reinterpret_cast<const void*>(sk_gemm_w4a16_kernel<SK_MODE_CLUSTER>)};
    for (int i = 0; i < 4 && r == cudaSuccess; ++i)
      r = cudaFuncSetAttribute(kernels[i], cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_LIMIT);
    return r;
  });
  if (e != cudaSuccess) return sk_set_cuda_error(e);
  const cudaStream_t cs = static_cast<cudaStream_t>(stream);
  __half* Ch = static_cast<__half*>(C);
  const bool pdl = (prob->flags & SK_FLAG_PDL) != 0;
  if (split)
    e = sk_launch(sk_gemm_w4a16_kernel<SK_MODE_CLUSTER>, p.sched.grid, NUM_THREADS, smem_bytes, cs, split, pdl,
                  tmA, qb, sz, Ch, p);
  else if (prob->schedule == SK_SCHED_DP)   // whole tiles only: no fixup code
    e = sk_launch(sk_gemm_w4a16_kernel<SK_EPI_WHOLE>, p.sched.grid, NUM_THREADS, smem_bytes, cs, 1, pdl,
                  tmA, qb, sz, Ch, p);
  else if (prob->fixup == SK_FIXUP_ATOMIC)
    e = sk_launch(sk_gemm_w4a16_kernel<SK_EPI_ATOMIC>, p.sched.grid, NUM_THREADS, smem_bytes, cs, 1, pdl,
                  tmA, qb, sz, Ch, p);
  else
    e = sk_launch(sk_gemm_w4a16_kernel<SK_EPI_BLOCK_REDUCE>, p.sched.grid, NUM_THREADS, smem_bytes, cs, 1, pdl,
                  tmA, qb, sz, Ch, p);
  if (e != cudaSuccess) return sk_set_cuda_error(e);
  return SK_OK;
}
