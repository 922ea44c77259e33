// fp16 Stream-K GEMM on sm_100a tensor cores: C[M,N] = A[M,K] . op(B),
// fp16 operands, fp32 accumulation in TMEM, fp16 result.
//
// Stands in for the TL kernels of streamk_fp16.py:116-373 (NT, explicit MMA),
// streamk_fp16_nn.py / streamk_fp16_nt.py (T.gemm), streamk_fp16_block_reduce.py
// and streamk_fp16_ladder*.py.  One persistent CTA per SM walks its share of
// tiles x K-iterations (sk_sched.h).  Inside a CTA three roles run in lock-step
// over the same segment list, synchronised by mbarriers only:
//
//   warps 0, 6  producers: TMA loads of the two operands' stage tiles (128-byte swizzle)
//   warp 1      MMA      : one thread issues tcgen05.mma, accumulators in TMEM
//                          (two buffers, so a segment's epilogue overlaps the
//                          next segment's mainloop)
//   warps 2..5  epilogue : tcgen05.ld -> fp16 store, or the cross-CTA fixup
//
// The reference's ldmatrix/mma.sync micro-kernel, its shared-memory swizzle and
// padding rules (streamk_fp16_block_reduce.py:82-110) and its intra-CTA split-K
// "block reduce" have no counterpart here: the tile K extent is fixed at 64
// halves (one 128-byte swizzle row), ragged edges are zero-filled by TMA, and
// TMEM accumulates over K.
#include "sk_common.cuh"
#include "sk_epilogue.cuh"

namespace {

using namespace skptx;

constexpr int BM = SK_BM;
constexpr int BK = 64;
constexpr int ROW_STAGE_BYTES = BM * BK * 2;   // 16 KB: 128 rows x 128 B
constexpr int NUM_THREADS = 256;   // warps: 0 row-operand producer, 1 MMA, 2..5 epilogue, 6 col-operand producer, 7 second MMA issuer
constexpr int MAX_STAGES = 12;
constexpr int CTRL_BYTES = 512;
constexpr int SMEM_LIMIT = 232448;             // 227 KB opt-in maximum per CTA

struct Ctrl {
  uint64_t full[MAX_STAGES];
  uint64_t empty[MAX_STAGES];
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

// Issue the loads of one operand's stage tile.  `first_row` is the tile's first row along
// the operand's MN extent, k the K iteration.
__device__ __forceinline__ void load_operand(int loader, uint32_t dst, const CUtensorMap* tm,
                                             const void* img, uint32_t bar, int first_row, int k,
                                             int tile_rows, int kblocks) {
  if (loader == SK_LOAD_TMA_K) {
    tma_load_2d(dst, tm, bar, k * BK, first_row);
  } else if (loader == SK_LOAD_TMA_MN) {
    for (int j = 0; j < tile_rows / 64; ++j) tma_load_2d(dst + j * 8192, tm, bar, first_row + j * 64, k * BK);
  } else {
    // pre-laid-out image: blocks of 128 rows x 64 halves, [row_block][k_block]
    const __half* src = static_cast<const __half*>(img);
    for (int j = 0; j < tile_rows / 128; ++j) {
      const size_t blk = static_cast<size_t>(first_row / 128 + j) * kblocks + k;
      bulk_load_1d(dst + j * 16384, src + blk * (128 * 64), 16384, bar);
    }
  }
}

// MODE SK_MODE_CLUSTER: the kernel of SK_SCHED_CLUSTER (one segment per CTA, exchange through
// distributed shared memory); otherwise the persistent Stream-K / data-parallel kernel with one
// of the workspace fixups (SK_EPI_ATOMIC, SK_EPI_BLOCK_REDUCE) or, for the data-parallel
// schedule, none (SK_EPI_WHOLE).  Four instantiations, so that none carries another's code: on
// small problems the kernel runs for microseconds and every instruction-cache line it touches
// is a miss.
constexpr int SK_MODE_CLUSTER = 3;   // besides SK_EPI_ATOMIC, SK_EPI_BLOCK_REDUCE, SK_EPI_WHOLE

template <int MODE>
__global__ void __launch_bounds__(NUM_THREADS, 1)
sk_gemm_f16_kernel(const __grid_constant__ CUtensorMap tmRow, const __grid_constant__ CUtensorMap tmCol,
                   const __grid_constant__ CUtensorMap tmC, __half* __restrict__ C, const SkParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;  // swizzle atoms need 1024-byte alignment
  uint8_t* smem = smem_raw + (base - raw_addr);
  const int STAGES = p.stages;
  const int G = p.kgroup;               // K steps per pipeline stage
  const uint32_t sRow = base;
  const uint32_t sCol = base + STAGES * G * ROW_STAGE_BYTES;
  Ctrl* ctrl = reinterpret_cast<Ctrl*>(smem + STAGES * G * (ROW_STAGE_BYTES + p.col_stage_bytes));
  volatile uint32_t* abort_flag = &ctrl->abort;

  // The single-thread roles (producers, MMA issuers) are run by their whole warp, with only the
  // TMA / tcgen05 / mbarrier instructions behind an elected lane (skptx::elect_one): the code
  // then is warp-uniform for the compiler, operands sit in uniform registers, and issuing one of
  // those instructions costs the warp about half of what it costs a lone lane inside a divergent
  // `if (lane == 0)` region (measured on the W4A16 kernel: 125 -> 65 cycles per UMMA).  The
  // warp index is therefore computed in the form the compiler knows to be uniform.  The cluster
  // instantiation keeps the plain form and single-lane loops: with the uniform form the W4A16
  // kernel's cluster start-up barrier never completed (cause not found by reading).
  constexpr bool clustered = MODE == SK_MODE_CLUSTER;
  const int warp = clustered ? static_cast<int>(threadIdx.x >> 5) : uniform_warp_idx();
  const int lane = threadIdx.x & 31;
  const int pid = blockIdx.x;
  const SkSched& s = p.sched;
  if (threadIdx.x == 0) {
    sk_trace(p, 0);
    griddep_launch_dependents();   // the next kernel of the stream may begin its own start-up
  }
  // Split-K inside a cluster: the partial tiles meet in a receive buffer behind the control block.
  const uint32_t recv_base = smem_u32(ctrl) + CTRL_BYTES;

  // Start-up.  The time from kernel entry to the first load is pure latency on every small
  // problem, and a lone thread retires a dependent instruction only every few cycles, so the
  // work is spread: an epilogue warp (idle until the first tile is done) initialises the
  // mbarriers, one per lane; meanwhile the producer and MMA threads work out their first
  // segment.  The producers then wait for nothing but the mbarriers (named barrier
  // BAR_PRODUCERS); the tensor-memory allocation runs beside the first loads and is awaited
  // by the MMA and epilogue warps only (BAR_CONSUMERS).
  constexpr int BAR_PRODUCERS = 2, BAR_CONSUMERS = 3;
  if (threadIdx.x == 0 && p.row_loader != SK_LOAD_IMAGE) prefetch_tensormap(&tmRow);
  if (threadIdx.x == 6 * 32 && p.col_loader != SK_LOAD_IMAGE) prefetch_tensormap(&tmCol);
  if (warp == 2) {
    if (lane < STAGES) {
      mbar_init(smem_u32(&ctrl->full[lane]), 1);
      mbar_init(smem_u32(&ctrl->empty[lane]), p.acc_b_off ? 2 : 1);   // MMA commit (+ the other issuer's "seen it")
    } else if (lane < STAGES + 2) {
      const int i = lane - STAGES;
      mbar_init(smem_u32(&ctrl->tmem_full[i]), p.acc_b_off ? 2 : 1);   // one arrival per MMA issuer
      mbar_init(smem_u32(&ctrl->tmem_empty[i]), 4);  // one arrival per epilogue warp
    } else if (lane == STAGES + 2) {
      if (clustered) mbar_init(smem_u32(&ctrl->recv_full), 5);   // 4 epilogue warps + the byte count
      ctrl->abort = 0u;
      ctrl->bcast = 0u;
      ctrl->pend[0].tile = -1;
      ctrl->pend[1].tile = -1;
    }
    fence_mbar_init();
    fence_proxy_async_smem();
    __syncwarp();
    named_bar_arrive(BAR_PRODUCERS, 96);      // warps 0 and 6 wait on it
    if (clustered && lane == STAGES + 2)
      mbar_arrive_expect_tx(smem_u32(&ctrl->recv_full),
                            static_cast<uint32_t>((s.split - 1) * p.cl_per) * SK_CL_QUAD_BYTES);
  }
  // first segment of this CTA, for the threads that walk the segment list from the start
  SkCursor cur;
  SkSeg seg;
  bool have = false;
  int tr = 0, tc = 0;
  const bool solo = clustered ? lane == 0 : true;   // which lanes of a single-thread role's warp run its loop
  if (solo && (warp == 0 || warp == 1 || warp == 6 || warp == 7)) {
    sk_cursor_init(s, pid, cur);
    have = sk_next(s, pid, cur, seg);
    if (have) sk_tile_mn(s, seg.tile, tr, tc);
  }
  // While the mbarriers are still being set up (and, with SK_FLAG_PDL, while the previous
  // kernel of the stream is still running) the producers already ask L2 for the boxes of their
  // first stages: the loads proper then find them there or on their way.
  if (lane == 0 && (warp == 0 || warp == 6) && have) {
    const bool is_row = warp == 0;
    if ((is_row ? p.row_loader : p.col_loader) == SK_LOAD_TMA_K) {
      const CUtensorMap* tm = is_row ? &tmRow : &tmCol;
      const int first_row = is_row ? tr * p.bm : tc * p.bn;
      int n = seg.k1 - seg.k0;
      if (n > STAGES * G) n = STAGES * G;
      if (n > p.prefetch_steps) n = p.prefetch_steps;
      for (int j = 0; j < n; ++j) tma_prefetch_2d(tm, (seg.k0 + j) * BK, first_row);
    }
  }
  uint32_t tmem_base = 0;
  if (warp == 0 || warp == 6) {
    named_bar_sync(BAR_PRODUCERS, 96);
  } else {
    if (warp == 1) {
      tmem_alloc(smem_u32(&ctrl->tmem_base), p.tmem_cols);
      tmem_relinquish();
    }
    tc_fence_before();
    named_bar_sync(BAR_CONSUMERS, NUM_THREADS - 64);   // warps 1..5 and 7
    tc_fence_after();
    tmem_base = *reinterpret_cast<volatile uint32_t*>(&ctrl->tmem_base);
  }
  if (threadIdx.x == 0) sk_trace(p, 1);
  // Everything up to here touched only this CTA's shared and tensor memory; global memory is
  // the previous kernel's until it has completed (a no-op unless launched with SK_FLAG_PDL).
  griddep_wait();

  if (warp == 0 || warp == 6) {
    // ------------------------------------------------------------- producers
    // Issuing a TMA instruction costs its thread tens of nanoseconds, and for narrow tiles
    // that, not bandwidth, bounds the K-step rate.  So two threads in two warps share the
    // work: warp 0 loads the row operand (and announces the stage's byte count), warp 6 the
    // column operand.  Both wait on the same "stage free" barrier.
    if (solo) {
      const bool leader = clustered ? true : elect_one();
      const bool is_row = warp == 0;
      bool traced = false;
      bool arrived = false;
      bool first_seg = true;
      int stage = 0;
      uint32_t ph = 0;
      bool ok = true;
      const uint32_t tx = p.row_tx_bytes + p.col_tx_bytes;
      const int loader = is_row ? p.row_loader : p.col_loader;
      const CUtensorMap* tm = is_row ? &tmRow : &tmCol;
      const void* img = is_row ? p.row_img : p.col_img;
      const int stage_bytes = is_row ? ROW_STAGE_BYTES : p.col_stage_bytes;
      const uint32_t dst0 = is_row ? sRow : sCol;
      const int tile_rows = is_row ? BM : p.bn;
      const uint32_t full0 = smem_u32(&ctrl->full[0]), empty0 = smem_u32(&ctrl->empty[0]);
      for (; ok && have; have = sk_next(s, pid, cur, seg)) {
        if (!first_seg) sk_tile_mn(s, seg.tile, tr, tc);   // (the first segment's are known already)
        first_seg = false;
        const int first_row = is_row ? tr * p.bm : tc * p.bn;
        for (int k = seg.k0; k < seg.k1;) {
          // up to G consecutive K steps share one stage: one barrier round trip for all
          const int n = (seg.k1 - k) < G ? (seg.k1 - k) : G;
          const uint32_t full = full0 + 8u * stage;
          if (!sk_wait_bar(empty0 + 8u * stage, ph ^ 1u, abort_flag, p, stage, is_row ? 0 : 4)) {
            ok = false;
            break;
          }
          if (leader) {
            if (is_row) mbar_arrive_expect_tx(full, n * tx);
            for (int j = 0; j < n; ++j) {
              const uint32_t dst = dst0 + (stage * G + j) * stage_bytes;
              if (loader == SK_LOAD_TMA_K) tma_load_2d(dst, tm, full, (k + j) * BK, first_row);
              else load_operand(loader, dst, tm, img, full, first_row, k + j, tile_rows, s.iters_per_tile);
            }
          }
          k += n;
          if (++stage == STAGES) {
            stage = 0; ph ^= 1u;
            // the ring is full for the first time: a good moment for this thread's share of
            // the cluster's start-up barrier
            // (thread 0 initialised the mbarriers the other CTAs will signal: it releases)
            if (clustered && !arrived) {
              if (is_row) cluster_arrive(); else cluster_arrive_relaxed();
              arrived = true;
            }
          }
          if (leader && is_row && !traced) { sk_trace(p, 2); traced = true; }
        }
      }
      if (clustered && !arrived) {
        if (is_row) cluster_arrive(); else cluster_arrive_relaxed();
      }
    } else if (clustered) {
      cluster_arrive_relaxed();
    }
  } else if (warp == 1 || warp == 7) {
    // ------------------------------------------------------------- MMA issuers
    // Issuing a UMMA costs its thread about 50 ns whatever the tile width, which bounds the
    // K-step rate of narrow tiles.  With room in tensor memory for two accumulators per
    // buffer (p.acc_b_off), a second thread in a warp of another scheduler takes every other
    // stage of a segment and accumulates on its own; the epilogue adds the two.
    const uint32_t me = warp == 1 ? 0u : 1u;
    if (solo && (me == 0u || p.acc_b_off != 0)) {
      const bool leader = clustered ? true : elect_one();
      const bool dual = p.acc_b_off != 0;
      int stage = 0;
      uint32_t ph = 0;
      uint32_t nseg = 0;
      bool ok = true;
      bool arrived = false;
      // K-major operand: 8-row groups 1024 B apart, 16 halves of K = 32 B.
      // MN-major operand: 64-wide chunks 8192 B apart, 8-row K groups 1024 B apart,
      // 16 rows of K = 2048 B.
      const bool row_mn = p.row_loader == SK_LOAD_TMA_MN;
      const bool col_mn = p.col_loader == SK_LOAD_TMA_MN;
      const uint32_t row_kstep16 = (row_mn ? 2048u : 32u) >> 4, col_kstep16 = (col_mn ? 2048u : 32u) >> 4;
      const uint64_t row_hi = umma_desc_sw128_hi(row_mn ? 8192u : 16u, 1024);
      const uint64_t col_hi = umma_desc_sw128_hi(col_mn ? 8192u : 16u, 1024);
      const uint32_t row_lo0 = umma_desc_lo(sRow), col_lo0 = umma_desc_lo(sCol);
      const uint32_t col_stage16 = static_cast<uint32_t>(p.col_stage_bytes) >> 4;
      const uint32_t idesc = p.idesc;
      const uint32_t full0 = smem_u32(&ctrl->full[0]), empty0 = smem_u32(&ctrl->empty[0]);
      const uint32_t acc_stride = p.acc_stride;
      for (; ok && have; have = sk_next(s, pid, cur, seg)) {
        const uint32_t buf = nseg & 1u;
        const uint32_t acc_ph = (nseg >> 1) & 1u;
        if (!sk_wait_bar(smem_u32(&ctrl->tmem_empty[buf]), acc_ph ^ 1u, abort_flag, p, 16 + buf, 1))
          break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * acc_stride + me * p.acc_b_off;
        uint32_t accumulate = 0u;   // this thread's first UMMA of the segment overwrites its accumulator
        uint32_t si = 0;            // stage number inside the segment
        for (int k = seg.k0; k < seg.k1; ++si) {
          const int n = (seg.k1 - k) < G ? (seg.k1 - k) : G;
          // Both issuers watch every stage's barrier complete, in order: a parity wait only
          // tells a phase from its neighbours, and loads may land out of order, so a thread
          // that skipped the other's stages could take a slot's previous use for the one it
          // waits for.
          if (!sk_wait_bar(full0 + 8u * stage, ph, abort_flag, p, 32 + stage, 1)) {
            ok = false;
            break;
          }
          if (dual && (si & 1u) != me) {   // the other issuer's stage
            // The slot must not be refilled before BOTH issuers have seen this use of it: a
            // lagging issuer that found the barrier two phases on would read that as "not yet"
            // and wait for a use that may never come.  So the skipping issuer arrives as well.
            if (leader) mbar_arrive(empty0 + 8u * stage);
            k += n;
            if (++stage == STAGES) { stage = 0; ph ^= 1u; }
            continue;
          }
          tc_fence_after();
          if (leader && nseg == 0 && k == seg.k0) sk_trace(p, 3);
          for (int j = 0; j < n; ++j) {
            const uint32_t a_lo = row_lo0 + (stage * G + j) * (ROW_STAGE_BYTES >> 4);
            const uint32_t b_lo = col_lo0 + (stage * G + j) * col_stage16;
#pragma unroll
            for (int kk = 0; kk < BK / 16; ++kk) {
              if (leader)
                umma_f16_ss(d_tmem, row_hi | (a_lo + kk * row_kstep16), col_hi | (b_lo + kk * col_kstep16),
                            idesc, accumulate);
              accumulate = 1u;
            }
          }
          if (leader) umma_commit(empty0 + 8u * stage);  // frees the stage when the MMAs retire
          k += n;
          if (++stage == STAGES) { stage = 0; ph ^= 1u; }
          // start-up barrier of the cluster: while the pipeline is still filling
          if (clustered && !arrived) { cluster_arrive_relaxed(); arrived = true; }
        }
        if (!ok) break;
        // (an issuer that issued nothing in this segment has nothing to wait for)
        if (leader) {
          if (accumulate) umma_commit(smem_u32(&ctrl->tmem_full[buf]));
          else mbar_arrive(smem_u32(&ctrl->tmem_full[buf]));
        }
        ++nseg;
      }
      if (leader && me == 0u) sk_trace(p, 4);
      if (clustered && !arrived) cluster_arrive_relaxed();
    } else if (clustered) {
      cluster_arrive_relaxed();
    }
  } else if (warp >= 2 && warp < 6) {
    // ------------------------------------------------------------- epilogue
    if constexpr (clustered)   // (takes part in the cluster's start-up barrier on its own)
      sk_cluster_send(p, static_cast<int>(cluster_ctarank()), warp, lane, tmem_base,
                      smem_u32(&ctrl->tmem_full[0]), sRow, recv_base, smem_u32(&ctrl->recv_full),
                      abort_flag, sk_cta_begin(s, pid) % s.iters_per_tile,
                      sk_cta_begin(s, pid + 1) - sk_cta_begin(s, pid));
    else
      sk_epilogue_loop<MODE>(p, C, pid, 0, warp, lane, tmem_base, smem_u32(&ctrl->tmem_full[0]),
                             smem_u32(&ctrl->tmem_empty[0]), &ctrl->bcast, abort_flag, ctrl->pend, &tmC,
                             p.c_tma ? smem_u32(ctrl) + 1024u : 0u);   // staging behind the control block
  }

  // ------------------------------------------------------------- teardown
  tc_fence_before();
  bool reduce_ok = true;
  if constexpr (clustered) {
    if (!(warp >= 2 && warp < 6)) cluster_wait();   // start-up barrier, second half
    __syncwarp();
    // the chunks of the other CTAs, and the epilogue warps' own one
    if (threadIdx.x == 0) sk_trace(p, 11);
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
      // A wait ran out: give copies and MMAs still in flight time to land before
      // the tensor memory goes back (bounded, no barrier to wait on any more).
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
    if (threadIdx.x == 0) sk_trace(p, 12);
    cluster_wait();
  } else {
    // Block-reduce fixup: every thread of the CTA now helps to reduce this CTA's slices of
    // the split tiles it took part in.
    if constexpr (MODE == SK_EPI_BLOCK_REDUCE) sk_reduce_pending(p, C, pid, 0, ctrl->pend, ctrl->ok);
  }
  if (threadIdx.x == 32) sk_trace(p, 7);
}

// ---------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_tiled() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess)
      return nullptr;
    if (q != cudaDriverEntryPointSuccess) return nullptr;
    return reinterpret_cast<EncodeTiledFn>(f);
  }();
  return fn;
}

}  // namespace

// fp16 row-major [rows, cols] tensor map with a {box_cols, box_rows} box and
// 128-byte swizzle; out-of-range elements read as zero.  L2 promotion 256 B: the next K step
// wants the neighbouring 128 bytes of every row (measured 1-3 % over 128 B).
int sk_make_tmap_f16(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols,
                     uint64_t ld_elems, uint32_t box_cols, uint32_t box_rows) {
  EncodeTiledFn enc = get_encode_tiled();
  if (!enc) return SK_ERR_LAUNCH;
  cuuint64_t gdim[2] = {cols, rows};
  cuuint64_t gstride[1] = {ld_elems * 2};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), gdim, gstride,
                   box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return sk_set_driver_error(static_cast<int>(r));
  return SK_OK;
}

// Fields of SkParams that depend only on the tile width: TMEM layout and pipeline depth.
void sk_fill_tile_params(SkParams* p, int bn, int stage_fixed_bytes, int max_stages,
                         int reserved_bytes, bool two_issuers) {
  p->bn = bn;
  const int acc_cols = (bn + 31) & ~31;
  // two accumulators per buffer when the kernel has two MMA issuers and tensor memory has room
  const bool dual = two_issuers && 4 * acc_cols <= 512;
  p->acc_b_off = dual ? acc_cols : 0;
  p->acc_stride = dual ? 2 * acc_cols : acc_cols;
  int cols = 32;
  while (cols < 2 * p->acc_stride) cols <<= 1;
  p->tmem_cols = cols;
  p->col_stage_bytes = bn * 128;
  int stages = (SMEM_LIMIT - 1024 - CTRL_BYTES - reserved_bytes) / (stage_fixed_bytes + p->col_stage_bytes);
  if (stages > max_stages) stages = max_stages;
  p->stages = stages;
}

int sk_launch_f16_2cta(const sk_problem* prob, const void* A, const void* B, void* C, SkParams* p,
                       void* const* peer_c, int n_peers, void* stream);

static int gemm_f16(const sk_problem* prob, const void* A, const void* B, void* C, void* const* peer_c,
                    int n_peers, void* ws, size_t ws_bytes, void* stream) {
  if (!prob || !A || !B || !C) return SK_ERR_ARG;
  if (prob->layout < SK_LAYOUT_NN || prob->layout > SK_LAYOUT_LADDER) return SK_ERR_ARG;
  if (prob->fixup != SK_FIXUP_ATOMIC && prob->fixup != SK_FIXUP_BLOCK_REDUCE) return SK_ERR_ARG;
  int num_sms = 0, dev_sms = 0;
  int st = sk_resolve_grid(prob, &num_sms, &dev_sms);
  if (st != SK_OK) return st;
  sk_problem resolved;   // SK_SCHED_AUTO -> a concrete schedule and tile, and the kernel to run
  int kind = 1, units = num_sms;
  sk_problem asked = *prob;
  if (n_peers < 0) {
    // fused reduce-scatter: the CTA-pair kernel, whole tiles (nothing of the partial product
    // stays on this GPU to fix up), C unused
    if (asked.tile_m != 0 && asked.tile_m != 256) return SK_ERR_ARG;
    asked.tile_m = 256;
    asked.schedule = SK_SCHED_DP;
    asked.ldc = asked.N;
  }
  sk_f16_dispatch(&asked, num_sms, n_peers > 0 ? n_peers : 0, &resolved, &kind, &units);
  if (n_peers < 0 && kind != 3) return SK_ERR_SHAPE;
  prob = &resolved;
  SkParams p;
  memset(&p, 0, sizeof(p));
  SkPlan plan;
  const bool pairs = kind == 3;
  // (pairs: tile_m 256 = asked for by the caller, 0 = the library's own choice)
  st = sk_make_sched(prob, kind, units, nullptr, &p.sched, &plan);
  if (st != SK_OK) return st;
  const int layout = prob->layout;
  const int M = prob->M, N = prob->N, K = prob->K;
  if (prob->lda < K || prob->ldc < N) return SK_ERR_SHAPE;
  if (layout == SK_LAYOUT_NT && prob->ldb < K) return SK_ERR_SHAPE;
  if (layout == SK_LAYOUT_NN && prob->ldb < N) return SK_ERR_SHAPE;
  // TMA: 16-byte aligned bases, row pitches multiples of 16 bytes.
  if ((reinterpret_cast<uintptr_t>(A) & 15u) || (reinterpret_cast<uintptr_t>(B) & 15u))
    return SK_ERR_ALIGN;
  if ((prob->lda & 7) != 0) return SK_ERR_ALIGN;
  if (layout != SK_LAYOUT_LADDER && (prob->ldb & 7) != 0) return SK_ERR_ALIGN;
  if ((reinterpret_cast<uintptr_t>(C) & 1u) != 0) return SK_ERR_ALIGN;
  if (!ws || ws_bytes < sk_ws_total_bytes(dev_sms)) return SK_ERR_WORKSPACE;
  if ((reinterpret_cast<uintptr_t>(ws) & 255u) != 0) return SK_ERR_ALIGN;
  if (prob->schedule == SK_SCHED_GEMV) {   // small M: the CUDA-core path (sk_gemv.cu)
    if (n_peers != 0) return SK_ERR_SHAPE;
    return sk_launch_gemv_f16(prob, A, B, C, sk_ws_carve(ws, dev_sms), num_sms, dev_sms, stream);
  }

  p.M = M; p.N = N; p.K = K;
  p.lda = prob->lda; p.ldb = prob->ldb; p.ldc = prob->ldc;
  p.rows = plan.rows; p.cols = plan.cols;
  p.transposed = plan.swap;
  p.unit_ctas = 1;
  p.bm = plan.bm;
  p.fixup = prob->fixup;
  p.c_vec_ok = ((reinterpret_cast<uintptr_t>(C) & 15u) == 0 && (prob->ldc & 7) == 0) ? 1 : 0;
  p.out_bf16 = (prob->flags & SK_FLAG_BF16) ? 1 : 0;
  p.drop_flag_cta = prob->test_drop_flag_cta - 1;
  p.timeout_ns = (prob->fixup_timeout_us > 0 ? static_cast<unsigned long long>(prob->fixup_timeout_us)
                                             : 2000000ULL) * 1000ULL;
  p.ws = sk_ws_carve(ws, dev_sms);  // layout fixed per device, whatever the grid
  p.trace = sk_trace_buffer();
  if (pairs) {
    p.bn = plan.bn;
    return sk_launch_f16_2cta(prob, A, B, C, &p, peer_c, n_peers, stream);
  }
  if (n_peers > 0) return SK_ERR_SHAPE;   // the fused all-gather lives in the CTA-pair kernel
  const int split = p.sched.split;   // SK_SCHED_CLUSTER: CTAs per tile
  // Whole tiles of a row-major C leave through shared memory and TMA stores (not the
  // transposed store of the swapped order, not the cluster schedule's reduction).
  p.c_tma = (!plan.swap && !split && p.c_vec_ok) ? 1 : 0;
  const int recv_bytes = split ? sk_cluster_recv_bytes(plan.bn, split) : p.c_tma ? 512 + SK_CSTAGE_BYTES : 0;
  p.cl_per = split ? sk_cluster_quads_per_cta(plan.bn, split) : 1;
  p.cl_per_div = sk_div_make(p.cl_per);
  sk_fill_tile_params(&p, plan.bn, ROW_STAGE_BYTES, MAX_STAGES, recv_bytes, true);
  if (p.stages < 2) return SK_ERR_SHAPE;
  // the staging area of the cluster exchange lives in the operand ring
  if (split && p.stages * (ROW_STAGE_BYTES + p.col_stage_bytes) < recv_bytes) return SK_ERR_SHAPE;
  // Very narrow tiles walked in long runs of K (data-parallel, or split over a cluster) are
  // bounded by the per-stage barrier round trip of the issuing threads, not by bandwidth: two
  // or four K steps then share a stage, which also asks DRAM for 256 or 512 contiguous bytes
  // of a weight row at a time.  Measured: 1.1-1.3x there.  Stream-K segments are short and
  // lose from the coarser stages, and so do wide tiles (few stages): one K step per stage.
  const bool long_runs = prob->schedule == SK_SCHED_DP || prob->schedule == SK_SCHED_CLUSTER;
  p.kgroup = !long_runs ? 1 : p.stages >= 12 ? 4 : p.stages >= 8 ? 2 : 1;
  p.stages /= p.kgroup;

  // Which matrix feeds which side of the UMMA.  Activations A are always K-major; the
  // weight operand is K-major (NT), MN-major (NN) or a pre-laid-out image (LADDER).
  const int w_loader = layout == SK_LAYOUT_NT ? SK_LOAD_TMA_K
                     : layout == SK_LAYOUT_NN ? SK_LOAD_TMA_MN : SK_LOAD_IMAGE;
  CUtensorMap tmRow, tmCol;
  memset(&tmRow, 0, sizeof(tmRow));
  memset(&tmCol, 0, sizeof(tmCol));
  auto weight_map = [&](CUtensorMap* tm, int tile_rows) -> int {
    if (layout == SK_LAYOUT_NT) return sk_make_tmap_f16(tm, B, N, K, prob->ldb, BK, tile_rows);
    if (layout == SK_LAYOUT_NN) return sk_make_tmap_f16(tm, B, K, N, prob->ldb, 64, BK);
    return SK_OK;
  };
  if (!plan.swap) {
    p.row_loader = SK_LOAD_TMA_K;
    p.col_loader = w_loader;
    st = sk_make_tmap_f16(&tmRow, A, M, K, prob->lda, BK, plan.bm);
    if (st == SK_OK) st = weight_map(&tmCol, plan.bn);
    p.col_img = B;
    if (w_loader != SK_LOAD_TMA_K && (plan.bn % 128) != 0) return SK_ERR_ARG;
  } else {
    p.row_loader = w_loader;
    p.col_loader = SK_LOAD_TMA_K;
    st = weight_map(&tmRow, plan.bm);
    if (st == SK_OK) st = sk_make_tmap_f16(&tmCol, A, M, K, prob->lda, BK, plan.bn);
    p.row_img = B;
  }
  if (st != SK_OK) return st;
  CUtensorMap tmC;
  memset(&tmC, 0, sizeof(tmC));
  if (p.c_tma) {
    st = sk_make_tmap_f16(&tmC, C, M, N, prob->ldc, 64, 32);
    if (st != SK_OK) return st;
  }
  p.row_tx_bytes = plan.bm * BK * 2;   // the TMA box of the M-side operand has plan.bm rows
  p.col_tx_bytes = p.col_stage_bytes;
  p.idesc = umma_idesc_f16(BM, plan.bn, 0, p.out_bf16) |
            (p.row_loader == SK_LOAD_TMA_MN ? (1u << 15) : 0u) |
            (p.col_loader == SK_LOAD_TMA_MN ? (1u << 16) : 0u);

  // Early L2 prefetch: up to six K steps, fewer for wide tiles (about 96 KB per producer;
  // measured: 2-5 % on the 10-20 us shapes, neutral to slightly negative beyond that budget).
  {
    const int box = p.row_tx_bytes > p.col_tx_bytes ? p.row_tx_bytes : p.col_tx_bytes;
    int n = box > 0 ? 98304 / box : 6;
    p.prefetch_steps = n > 6 ? 6 : n < 2 ? 2 : n;
  }
  const int smem_bytes =
      p.stages * p.kgroup * (ROW_STAGE_BYTES + p.col_stage_bytes) + 1024 + CTRL_BYTES + recv_bytes;
  static SkPerDeviceOnce attrs;
  cudaError_t e = attrs.run([]() {
    cudaError_t r = cudaSuccess;
    const void* kernels[4] = {
        reinterpret_cast<const void*>(sk_gemm_f16_kernel<SK_EPI_ATOMIC>),
        reinterpret_cast<const void*>(sk_gemm_f16_kernel<SK_EPI_BLOCK_REDUCE>),
        reinterpret_cast<const void*>(sk_gemm_f16_kernel<SK_EPI_WHOLE>),
        reinterpret_cast<const void*>(sk_gemm_f16_kernel<SK_MODE_CLUSTER>)};
    for (int i = 0; i < 4 && r == cudaSuccess; ++i)
      r = cudaFuncSetAttribute(kernels[i], cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_LIMIT);
    return r;
  });
  if (e != cudaSuccess) return sk_set_cuda_error(e);
  const cudaStream_t cs = static_cast<cudaStream_t>(stream);
  __half* Ch = static_cast<__half*>(C);
  const bool pdl = (prob->flags & SK_FLAG_PDL) != 0;
  if (split)
    e = sk_launch(sk_gemm_f16_kernel<SK_MODE_CLUSTER>, p.sched.grid, NUM_THREADS, smem_bytes, cs, split, pdl,
                  tmRow, tmCol, tmC, Ch, p);
  else if (prob->schedule == SK_SCHED_DP)   // whole tiles only: no fixup code
    e = sk_launch(sk_gemm_f16_kernel<SK_EPI_WHOLE>, p.sched.grid, NUM_THREADS, smem_bytes, cs, 1, pdl,
                  tmRow, tmCol, tmC, Ch, p);
  else if (prob->fixup == SK_FIXUP_ATOMIC)
    e = sk_launch(sk_gemm_f16_kernel<SK_EPI_ATOMIC>, p.sched.grid, NUM_THREADS, smem_bytes, cs, 1, pdl,
                  tmRow, tmCol, tmC, Ch, p);
  else
    e = sk_launch(sk_gemm_f16_kernel<SK_EPI_BLOCK_REDUCE>, p.sched.grid, NUM_THREADS, smem_bytes, cs, 1, pdl,
                  tmRow, tmCol, tmC, Ch, p);
  if (e != cudaSuccess) return sk_set_cuda_error(e);
  return SK_OK;
}

extern "C" int sk_gemm_f16(const sk_problem* prob, const void* A, const void* B, void* C, void* ws,
                           size_t ws_bytes, void* stream) {
  return gemm_f16(prob, A, B, C, nullptr, 0, ws, ws_bytes, stream);
}

extern "C" int sk_gemm_f16_scatter(const sk_problem* prob, const void* A, const void* B, void* const* dst,
                                   int n_blocks, void* ws, size_t ws_bytes, void* stream) {
  if (n_blocks < 1 || n_blocks > SK_MAX_TARGETS || !dst || !dst[0]) return SK_ERR_ARG;
  return gemm_f16(prob, A, B, dst[0], dst, -n_blocks, ws, ws_bytes, stream);
}

extern "C" int sk_gemm_f16_gather(const sk_problem* prob, const void* A, const void* B, void* C,
                                  void* const* peers, int n_peers, void* ws, size_t ws_bytes,
                                  void* stream) {
  if (n_peers < 0 || n_peers > SK_MAX_PEERS || (n_peers > 0 && !peers)) return SK_ERR_ARG;
  return gemm_f16(prob, A, B, C, peers, n_peers, ws, ws_bytes, stream);
}
