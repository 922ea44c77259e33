// fp16 Stream-K GEMM on sm_100a tensor cores: C[M,N] = A[M,K] . op(B),
// fp16 operands, fp32 accumulation in TMEM, fp16 result.
//
// Stands in for the TL kernels of streamk_fp16.py:116-373 (NT, explicit MMA),
// streamk_fp16_nn.py / streamk_fp16_nt.py (T.gemm), streamk_fp16_block_reduce.py
// and streamk_fp16_ladder*.py.  One persistent CTA per SM walks its share of
// tiles x K-iterations (sk_sched.h).  Inside a CTA three roles run in lock-step
// over the same segment list, synchronised by mbarriers only:
//
//   warp 0      producer : TMA loads of the A and B stage tiles (128-byte swizzle)
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
constexpr int A_STAGE_BYTES = BM * BK * 2;
constexpr int NUM_THREADS = 192;

enum { BMODE_NT = 0, BMODE_NN = 1, BMODE_LADDER = 2 };

template <int BN>
struct Cfg {
  static constexpr int B_STAGE_BYTES = BN * BK * 2;
  static constexpr int STAGES = (BN == 128) ? 6 : 4;
  static constexpr int TMEM_COLS = 2 * BN;  // two fp32 accumulators of BN columns
  static constexpr int PIPE_BYTES = STAGES * (A_STAGE_BYTES + B_STAGE_BYTES);
  static constexpr int SMEM_BYTES = PIPE_BYTES + 1024 /*alignment slack*/ + 256 /*Ctrl*/;
};

struct Ctrl {
  uint64_t full[8];
  uint64_t empty[8];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  uint32_t abort;
  uint32_t bcast;
};
static_assert(sizeof(Ctrl) <= 256, "Ctrl must fit its reserved space");

template <int BN, int BMODE>
__global__ void __launch_bounds__(NUM_THREADS, 1)
sk_gemm_f16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                   const __half* __restrict__ Bimg, __half* __restrict__ C, const SkParams p) {
  using cfg = Cfg<BN>;
  constexpr int STAGES = cfg::STAGES;
  constexpr int B_STAGE_BYTES = cfg::B_STAGE_BYTES;
  constexpr uint32_t IDESC = umma_idesc_f16(BM, BN, BMODE == BMODE_NN ? 1 : 0);
  constexpr size_t SLOT_FLOATS = SK_SLOT_BYTES / sizeof(float);

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;  // swizzle atoms need 1024-byte alignment
  uint8_t* smem = smem_raw + (base - raw_addr);
  const uint32_t sA = base;
  const uint32_t sB = base + STAGES * A_STAGE_BYTES;
  Ctrl* ctrl = reinterpret_cast<Ctrl*>(smem + cfg::PIPE_BYTES);
  volatile uint32_t* abort_flag = &ctrl->abort;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int pid = blockIdx.x;
  const SkSched& s = p.sched;
  if (threadIdx.x == 0) sk_trace(p, 0);

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) {
      mbar_init(smem_u32(&ctrl->full[i]), 1);
      mbar_init(smem_u32(&ctrl->empty[i]), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&ctrl->tmem_full[i]), 1);
      mbar_init(smem_u32(&ctrl->tmem_empty[i]), 4);  // one arrival per epilogue warp
    }
    ctrl->abort = 0u;
    ctrl->bcast = 0u;
    fence_mbar_init();
    fence_proxy_async_smem();
    prefetch_tensormap(&tmA);
    if (BMODE != BMODE_LADDER) prefetch_tensormap(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&ctrl->tmem_base), cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&ctrl->tmem_base);
  if (threadIdx.x == 0) sk_trace(p, 1);

  if (warp == 0) {
    // ------------------------------------------------------------- producer
    if (lane == 0) {
      bool traced = false;
      SkCursor cur;
      sk_cursor_init(s, pid, cur);
      SkSeg seg;
      int stage = 0;
      uint32_t ph = 0;
      bool ok = true;
      while (ok && sk_next(s, pid, cur, seg)) {
        int tm, tn;
        sk_tile_mn(s, seg.tile, tm, tn);
        const int m0 = tm * BM, n0 = tn * BN;
        for (int k = seg.k0; k < seg.k1; ++k) {
          const uint32_t full = smem_u32(&ctrl->full[stage]);
          if (!sk_wait_bar(smem_u32(&ctrl->empty[stage]), ph ^ 1u, abort_flag, p, stage, 0)) {
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(full, p.a_tx_bytes + B_STAGE_BYTES);
          tma_load_2d(sA + stage * A_STAGE_BYTES, &tmA, full, k * BK, m0);
          const uint32_t dstB = sB + stage * B_STAGE_BYTES;
          if (BMODE == BMODE_NT) {
            tma_load_2d(dstB, &tmB, full, k * BK, n0);
          } else if (BMODE == BMODE_NN) {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(dstB + j * 8192, &tmB, full, n0 + j * 64, k * BK);
          } else {
            // pre-laid-out image: blocks of 128 rows x 64 halves, [n_block][k_block]
            const int kblocks = s.iters_per_tile;
#pragma unroll
            for (int j = 0; j < BN / 128; ++j) {
              const size_t blk = static_cast<size_t>(n0 / 128 + j) * kblocks + k;
              bulk_load_1d(dstB + j * 16384, Bimg + blk * (128 * 64), 16384, full);
            }
          }
          if (++stage == STAGES) { stage = 0; ph ^= 1u; }
          if (!traced) { sk_trace(p, 2); traced = true; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      SkCursor cur;
      sk_cursor_init(s, pid, cur);
      SkSeg seg;
      int stage = 0;
      uint32_t ph = 0;
      uint32_t nseg = 0;
      bool ok = true;
      while (ok && sk_next(s, pid, cur, seg)) {
        const uint32_t buf = nseg & 1u;
        const uint32_t acc_ph = (nseg >> 1) & 1u;
        if (!sk_wait_bar(smem_u32(&ctrl->tmem_empty[buf]), acc_ph ^ 1u, abort_flag, p, 16 + buf, 1))
          break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int k = seg.k0; k < seg.k1; ++k) {
          if (!sk_wait_bar(smem_u32(&ctrl->full[stage]), ph, abort_flag, p, 8 + stage, 1)) {
            ok = false;
            break;
          }
          tc_fence_after();
          if (nseg == 0 && k == seg.k0) sk_trace(p, 3);
          const uint32_t a_addr = sA + stage * A_STAGE_BYTES;
          const uint32_t b_addr = sB + stage * B_STAGE_BYTES;
#pragma unroll
          for (int kk = 0; kk < BK / 16; ++kk) {
            // K-major operand: 8-row groups 1024 B apart, 16 halves of K = 32 B.
            const uint64_t da = umma_desc_sw128(a_addr + kk * 32, 16, 1024);
            // MN-major B (NN layout): 64-column chunks 8192 B apart, 8-row K groups
            // 1024 B apart, 16 rows of K = 2048 B.
            const uint64_t db = (BMODE == BMODE_NN)
                                    ? umma_desc_sw128(b_addr + kk * 2048, 8192, 1024)
                                    : umma_desc_sw128(b_addr + kk * 32, 16, 1024);
            umma_f16_ss(d_tmem, da, db, IDESC, (k > seg.k0 || kk > 0) ? 1u : 0u);
          }
          umma_commit(smem_u32(&ctrl->empty[stage]));  // frees the stage when the MMAs retire
          if (++stage == STAGES) { stage = 0; ph ^= 1u; }
        }
        if (!ok) break;
        umma_commit(smem_u32(&ctrl->tmem_full[buf]));
        ++nseg;
      }
      sk_trace(p, 4);
    }
  } else {
    // ------------------------------------------------------------- epilogue
    sk_epilogue_loop<BN>(p, C, pid, warp, lane, tmem_base, smem_u32(&ctrl->tmem_full[0]),
                         smem_u32(&ctrl->tmem_empty[0]), &ctrl->bcast, abort_flag);
  }

  // ------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    if (*abort_flag) {
      // A wait ran out: give copies and MMAs still in flight time to land before
      // the tensor memory goes back (bounded, no barrier to wait on any more).
      const unsigned long long t0 = globaltimer_ns();
      while (globaltimer_ns() - t0 < 200000ULL) __nanosleep(1000);
    }
    tc_fence_after();
    __syncwarp();
    tmem_dealloc(tmem_base, cfg::TMEM_COLS);
    if (lane == 0) sk_trace(p, 7);
  }
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
// 128-byte swizzle; out-of-range elements read as zero.
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
                   CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    sk_set_cuda_error(cudaErrorInvalidValue);
    return SK_ERR_LAUNCH;
  }
  return SK_OK;
}

namespace {

template <int BN, int BMODE>
int launch_f16(const CUtensorMap& tmA, const CUtensorMap& tmB, const __half* Bimg, __half* C,
               const SkParams& p, cudaStream_t cs) {
  using cfg = Cfg<BN>;
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_set[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(sk_gemm_f16_kernel<BN, BMODE>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, cfg::SMEM_BYTES);
    if (e != cudaSuccess) return sk_set_cuda_error(e);
    attr_set[dev & 63] = true;
  }
  sk_gemm_f16_kernel<BN, BMODE><<<p.sched.grid, NUM_THREADS, cfg::SMEM_BYTES, cs>>>(tmA, tmB, Bimg, C, p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return sk_set_cuda_error(e);
  return SK_OK;
}

}  // namespace

extern "C" int sk_gemm_f16(const sk_problem* prob, const void* A, const void* B, void* C, void* ws,
                           size_t ws_bytes, void* stream) {
  if (!prob || !A || !B || !C) return SK_ERR_ARG;
  if (prob->layout < SK_LAYOUT_NN || prob->layout > SK_LAYOUT_LADDER) return SK_ERR_ARG;
  if (prob->fixup != SK_FIXUP_ATOMIC && prob->fixup != SK_FIXUP_BLOCK_REDUCE) return SK_ERR_ARG;
  int num_sms = 0, dev_sms = 0;
  int st = sk_resolve_grid(prob, &num_sms, &dev_sms);
  if (st != SK_OK) return st;
  SkParams p;
  memset(&p, 0, sizeof(p));
  sk_schedule_info info;
  st = sk_make_sched(prob, 1, num_sms, &info, &p.sched);
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

  p.M = M; p.N = N; p.K = K;
  p.lda = prob->lda; p.ldb = prob->ldb; p.ldc = prob->ldc;
  p.fixup = prob->fixup;
  p.c_vec_ok = ((reinterpret_cast<uintptr_t>(C) & 15u) == 0 && (prob->ldc & 7) == 0) ? 1 : 0;
  p.drop_flag_cta = prob->test_drop_flag_cta;
  p.timeout_ns = (prob->fixup_timeout_us > 0 ? static_cast<unsigned long long>(prob->fixup_timeout_us)
                                             : 2000000ULL) * 1000ULL;
  p.ws = sk_ws_carve(ws, dev_sms);  // layout fixed per device, whatever the grid
  p.trace = sk_trace_buffer();

  const int BN = info.tile_n;
  CUtensorMap tmA, tmB;
  memset(&tmB, 0, sizeof(tmB));
  // A short problem loads only the rows it has (rounded up to 8): the UMMA still reads 128
  // rows of the stage, the rest is stale shared memory feeding accumulator rows nobody reads.
  const int a_rows = M >= BM ? BM : ((M + 7) & ~7);
  p.a_tx_bytes = a_rows * BK * 2;
  st = sk_make_tmap_f16(&tmA, A, M, K, prob->lda, BK, a_rows);
  if (st != SK_OK) return st;
  if (layout == SK_LAYOUT_NT) {
    st = sk_make_tmap_f16(&tmB, B, N, K, prob->ldb, BK, BN);
  } else if (layout == SK_LAYOUT_NN) {
    st = sk_make_tmap_f16(&tmB, B, K, N, prob->ldb, 64, BK);
  }
  if (st != SK_OK) return st;

  cudaStream_t cs = static_cast<cudaStream_t>(stream);
  const __half* Bh = static_cast<const __half*>(B);
  __half* Ch = static_cast<__half*>(C);
  if (BN == 128) {
    if (layout == SK_LAYOUT_NT) return launch_f16<128, BMODE_NT>(tmA, tmB, Bh, Ch, p, cs);
    if (layout == SK_LAYOUT_NN) return launch_f16<128, BMODE_NN>(tmA, tmB, Bh, Ch, p, cs);
    return launch_f16<128, BMODE_LADDER>(tmA, tmB, Bh, Ch, p, cs);
  } else {
    if (layout == SK_LAYOUT_NT) return launch_f16<256, BMODE_NT>(tmA, tmB, Bh, Ch, p, cs);
    if (layout == SK_LAYOUT_NN) return launch_f16<256, BMODE_NN>(tmA, tmB, Bh, Ch, p, cs);
    return launch_f16<256, BMODE_LADDER>(tmA, tmB, Bh, Ch, p, cs);
  }
}
