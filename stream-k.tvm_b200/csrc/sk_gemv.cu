// Small-M path (SK_SCHED_GEMV, M <= 4): C[M,N] = A[M,K] . W^T on the CUDA cores.
//
// With one to four rows of activations a weight is used M times, the product is a stream of the
// weight matrix, and the tensor-core kernels spend more time on their fixed costs (tensor-memory
// allocation, mbarrier rings, a cluster exchange or a workspace fix-up: 6-8 us per launch) than
// the stream itself takes.  These kernels have none of that: a grid of several CTAs per SM, each
// thread keeping eight 16-byte loads of weights in flight, fp32 FMAs, and a split of K whose
// partial sums meet in the workspace and are added in split order by the last CTA of a row group
// to arrive (a counter tells), so the result is bitwise reproducible like the block-reduce
// fixup's.  The reference has no such path: its kernels are tiled for the tensor cores at every
// M (streamk_fp16.py:143-371, streamk_fp16_ladder_block_reduce_q4.py:143-522).
//
// Work split: a row group is 128 weight rows; CTA (g, s) walks K range s of group g.
//   fp16 / bf16 weights [N, K] row-major: a warp takes 16 rows, eight at a time; its 32 lanes read
//     512 contiguous bytes of one row per instruction (8 K values each), the activations of the
//     lane's K values sit in registers for all eight rows, and the lanes' sums meet in a
//     shuffle tree at the end.
//   W4A16 packed image (sk_prepack_q4: [row block][K block] of [half][row][16 B]): a thread owns
//     one weight row, reads its 2 x 16 bytes of a K block (a warp: 512 contiguous bytes each),
//     turns the nibbles into fp32 (q - z) with one logic and one add each, multiplies with
//     activations that every lane reads from the same shared-memory address, and applies the
//     scale once per scale group.
#include "sk_common.cuh"

namespace {

constexpr int GEMV_THREADS_F16 = 256;
constexpr int GEMV_THREADS_Q4 = 128;

__device__ __forceinline__ uint4 ld_stream_v4(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

template <bool BF16>
__device__ __forceinline__ void unpack2(uint32_t w, float& lo, float& hi) {
  if constexpr (BF16) {
    lo = __uint_as_float(w << 16);
    hi = __uint_as_float(w & 0xFFFF0000u);
  } else {
    const __half2 h = *reinterpret_cast<const __half2*>(&w);
    const float2 f = __half22float2(h);
    lo = f.x;
    hi = f.y;
  }
}

__device__ __forceinline__ uint32_t pack_out(float v, int bf16) {
  uint32_t r;
  if (bf16) asm("cvt.rn.bf16x2.f32 %0, %2, %1;" : "=r"(r) : "f"(v), "f"(0.f));
  else      asm("cvt.rn.f16x2.f32 %0, %2, %1;" : "=r"(r) : "f"(v), "f"(0.f));
  return r & 0xFFFFu;
}

// Activations of this CTA's K range as fp32 in shared memory: sA[m][k - k_lo], zero beyond K.
template <int M, bool BF16>
__device__ __forceinline__ void stage_activations(float* sA, const uint16_t* A, int lda, int K, int k_lo,
                                                  int k_len, int tid, int nthreads) {
  for (int i = tid; i < M * (k_len >> 3); i += nthreads) {
    const int m = i / (k_len >> 3), c = i - m * (k_len >> 3);
    const int k = k_lo + c * 8;
    float f[8];
    if (k < K) {   // (K is a multiple of 8: a chunk is inside or outside as a whole)
      const uint4 v = *reinterpret_cast<const uint4*>(A + static_cast<size_t>(m) * lda + k);
      unpack2<BF16>(v.x, f[0], f[1]);
      unpack2<BF16>(v.y, f[2], f[3]);
      unpack2<BF16>(v.z, f[4], f[5]);
      unpack2<BF16>(v.w, f[6], f[7]);
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) f[e] = 0.f;
    }
    float4* dst = reinterpret_cast<float4*>(sA + m * k_len + c * 8);
    dst[0] = make_float4(f[0], f[1], f[2], f[3]);
    dst[1] = make_float4(f[4], f[5], f[6], f[7]);
  }
}

// Partial sums of CTA (g, s) are at parts[((g * S + s) * M + m) * 128 + row]; the last CTA of
// group g to arrive adds them over s = 0 .. S-1 in that order and stores C[m][g * 128 + row].
template <int M>
__device__ __forceinline__ void finish_group(const float* sums /* shared: [M][128] */, float* parts,
                                             uint32_t* counters, uint16_t* C, int ldc, int N, int g, int s,
                                             int S, int bf16, int tid, int nthreads, uint32_t* s_last) {
  const int row0 = g * SK_GEMV_ROWS;
  if (S == 1) {
    for (int i = tid; i < M * SK_GEMV_ROWS; i += nthreads) {
      const int m = i >> 7, r = i & 127;
      if (row0 + r < N) C[static_cast<size_t>(m) * ldc + row0 + r] = static_cast<uint16_t>(pack_out(sums[i], bf16));
    }
    return;
  }
  float* mine = parts + static_cast<size_t>(g * S + s) * (M * SK_GEMV_ROWS);
  for (int i = tid; i < M * SK_GEMV_ROWS; i += nthreads) __stcg(mine + i, sums[i]);
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const uint32_t old = atomicAdd(counters + g, 1u);
    *s_last = old == static_cast<uint32_t>(S - 1) ? 1u : 0u;
  }
  __syncthreads();
  if (*s_last == 0u) return;
  __threadfence();
  const float* all = parts + static_cast<size_t>(g * S) * (M * SK_GEMV_ROWS);
  for (int i = tid; i < M * SK_GEMV_ROWS; i += nthreads) {
    const int m = i >> 7, r = i & 127;
    float acc = 0.f;
    for (int j0 = 0; j0 < S; j0 += 8) {     // eight loads in flight, added in split order
      float v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u)
        v[u] = __ldcg(all + static_cast<size_t>(j0 + u < S ? j0 + u : S - 1) * (M * SK_GEMV_ROWS) + i);
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (j0 + u < S) acc += v[u];
    }
    if (row0 + r < N) C[static_cast<size_t>(m) * ldc + row0 + r] = static_cast<uint16_t>(pack_out(acc, bf16));
  }
  if (tid == 0) counters[g] = 0u;   // zero between launches, like every counter of the workspace
}

// ------------------------------------------------------------------------------------- fp16
template <int M, bool BF16>
__global__ void __launch_bounds__(GEMV_THREADS_F16)
sk_gemv_f16_kernel(const uint16_t* __restrict__ A, int lda, const uint16_t* __restrict__ B, int ldb,
                   uint16_t* __restrict__ C, int ldc, int N, int K, int k_per_split, int S, float* parts,
                   uint32_t* counters) {
  extern __shared__ __align__(16) float sA[];   // [M][k_per_split]
  __shared__ float sums[M * SK_GEMV_ROWS];
  __shared__ uint32_t s_last;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = blockIdx.x / S, s = blockIdx.x - g * S;
  const int k_lo = s * k_per_split;
  skptx::griddep_wait();
  stage_activations<M, BF16>(sA, A, lda, K, k_lo, k_per_split, tid, GEMV_THREADS_F16);
  __syncthreads();
  int k_hi = k_lo + k_per_split;
  if (k_hi > K) k_hi = K;
#pragma unroll 1
  for (int batch = 0; batch < 2; ++batch) {
    const int r0 = g * SK_GEMV_ROWS + warp * 16 + batch * 8;
    float acc[8][M];
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int m = 0; m < M; ++m) acc[j][m] = 0.f;
    for (int k = k_lo + lane * 8; k < k_hi; k += 256) {
      uint4 w[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        // (rows past N repeat the last row: loaded, never stored)
        const int r = r0 + j < N ? r0 + j : N - 1;
        w[j] = ld_stream_v4(B + static_cast<size_t>(r) * ldb + k);
      }
      float a[M][8];
#pragma unroll
      for (int m = 0; m < M; ++m) {
        const float4* src = reinterpret_cast<const float4*>(sA + m * k_per_split + (k - k_lo));
        const float4 x = src[0], y = src[1];
        a[m][0] = x.x; a[m][1] = x.y; a[m][2] = x.z; a[m][3] = x.w;
        a[m][4] = y.x; a[m][5] = y.y; a[m][6] = y.z; a[m][7] = y.w;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float f[8];
        unpack2<BF16>(w[j].x, f[0], f[1]);
        unpack2<BF16>(w[j].y, f[2], f[3]);
        unpack2<BF16>(w[j].z, f[4], f[5]);
        unpack2<BF16>(w[j].w, f[6], f[7]);
#pragma unroll
        for (int m = 0; m < M; ++m)
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[j][m] = fmaf(f[e], a[m][e], acc[j][m]);
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int m = 0; m < M; ++m) {
        float v = acc[j][m];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (lane == 0) sums[m * SK_GEMV_ROWS + warp * 16 + batch * 8 + j] = v;
      }
  }
  // (SK_FLAG_PDL: the grid has several CTAs per SM, so the next kernel's CTAs are let in only
  // now, when this one needs its slot no longer; earlier they would take the slots of CTAs
  // of this grid that have not started)
  skptx::griddep_launch_dependents();
  __syncthreads();
  finish_group<M>(sums, parts, counters, C, ldc, N, g, s, S, BF16 ? 1 : 0, tid, GEMV_THREADS_F16, &s_last);
}

// ------------------------------------------------------------------------------------ W4A16
// Activations of this CTA's K range as fp16 in shared memory, sA[m][k - k_lo] (zero beyond K),
// each row multiplied by a power of two that brings its largest magnitude into [32, 64): the
// inner sums below are taken in fp16 over 16 terms of |q - z| <= 15, which then stay below
// 16 * 15 * 64 whatever the activations are (an outlier of a few thousand would overflow them
// otherwise).  inv[m] undoes the factor (exactly) on the fp32 side.
template <int M>
__device__ __forceinline__ void stage_activations_scaled(uint16_t* sA, float* s_max /* shared [M][4] */,
                                                         const uint16_t* A, int lda, int K, int k_lo, int k_len,
                                                         int tid, float (&inv)[M]) {
  const int chunks = k_len >> 3;   // 16-byte chunks per row; at most 2 per thread (k_len <= 2048)
  const int warp = tid >> 5, lane = tid & 31;
#pragma unroll
  for (int m = 0; m < M; ++m) {
    __half2 mx = __float2half2_rn(0.f);
    for (int c = tid; c < chunks; c += GEMV_THREADS_Q4) {
      const int k = k_lo + c * 8;
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (k < K) v = *reinterpret_cast<const uint4*>(A + static_cast<size_t>(m) * lda + k);
      *reinterpret_cast<uint4*>(sA + m * k_len + c * 8) = v;
      const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
      for (int e = 0; e < 4; ++e) mx = __hmax2(mx, __habs2(h[e]));
    }
    float f = fmaxf(__low2float(mx), __high2float(mx));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) f = fmaxf(f, __shfl_xor_sync(0xffffffffu, f, o));
    if (lane == 0) s_max[m * 4 + warp] = f;
  }
  __syncthreads();
#pragma unroll
  for (int m = 0; m < M; ++m) {
    const float f = fmaxf(fmaxf(s_max[m * 4], s_max[m * 4 + 1]), fmaxf(s_max[m * 4 + 2], s_max[m * 4 + 3]));
    int e = 132 - static_cast<int>((__float_as_uint(f) >> 23) & 0xFFu);   // 2^e * max in [32, 64)
    e = e < -11 ? -11 : (e > 14 ? 14 : e);                                 // 2^e is a normal fp16
    const __half2 up = __float2half2_rn(__uint_as_float(static_cast<uint32_t>(127 + e) << 23));
    inv[m] = __uint_as_float(static_cast<uint32_t>(127 - e) << 23);
    for (int c = tid; c < chunks; c += GEMV_THREADS_Q4) {   // (the chunks this thread wrote)
      uint4* dst = reinterpret_cast<uint4*>(sA + m * k_len + c * 8);
      uint4 v = *dst;
      __half2* h = reinterpret_cast<__half2*>(&v);
#pragma unroll
      for (int q = 0; q < 4; ++q) h[q] = __hmul2(h[q], up);
      *dst = v;
    }
  }
  __syncthreads();
}

// The eight nibbles of a packed word as four fp16 pairs (q - z), without a conversion
// instruction.  The word's low half holds the even K values of its eight and the high half the
// odd ones, so one mask picks a pair of neighbours: a nibble in bits 0-3 of 0x6400 reads as
// 1024 + q, in bits 4-7 as 1024 + 16 q; `c0` = 1024 + z, `c1` = -(64 + z): both results exact.
__device__ __forceinline__ void nibbles8(uint32_t w, __half2 c0, __half2 c1, __half2 (&d)[4]) {
  uint32_t t0, t1, t2, t3;
  const uint32_t w8 = w >> 8;
  asm("lop3.b32 %0, %1, 0x000F000F, 0x64006400, 0xEA;" : "=r"(t0) : "r"(w));
  asm("lop3.b32 %0, %1, 0x00F000F0, 0x64006400, 0xEA;" : "=r"(t1) : "r"(w));
  asm("lop3.b32 %0, %1, 0x000F000F, 0x64006400, 0xEA;" : "=r"(t2) : "r"(w8));
  asm("lop3.b32 %0, %1, 0x00F000F0, 0x64006400, 0xEA;" : "=r"(t3) : "r"(w8));
  const __half2 sixteenth = __float2half2_rn(0.0625f);
  d[0] = __hsub2(*reinterpret_cast<const __half2*>(&t0), c0);              // K values 0, 1
  d[1] = __hfma2(*reinterpret_cast<const __half2*>(&t1), sixteenth, c1);   //          2, 3
  d[2] = __hsub2(*reinterpret_cast<const __half2*>(&t2), c0);              //          4, 5
  d[3] = __hfma2(*reinterpret_cast<const __half2*>(&t3), sixteenth, c1);   //          6, 7
}

// A thread owns one weight row of the 128-row block; four K blocks (256 of K) per step: eight
// 16-byte loads per thread in flight, the first step's already while the activations are staged.
template <int M>
__global__ void __launch_bounds__(GEMV_THREADS_Q4)
sk_gemv_q4_kernel(const uint16_t* __restrict__ A, int lda, const uint8_t* __restrict__ qblocks,
                  const uint8_t* __restrict__ szblocks, uint16_t* __restrict__ C, int ldc, int N, int K,
                  int kblocks, int kb_per_split, int S, int gshift, int q_groups, float* parts,
                  uint32_t* counters) {
  extern __shared__ __align__(16) uint16_t sAh[];   // [M][kb_per_split * 64]
  __shared__ float sums[M * SK_GEMV_ROWS];
  __shared__ float s_max[M * 4];
  __shared__ uint32_t s_last;
  const int tid = threadIdx.x;                // = weight row inside the 128-row block
  const int g = blockIdx.x / S, s = blockIdx.x - g * S;
  const int kb_lo = s * kb_per_split;
  int kb_hi = kb_lo + kb_per_split;
  if (kb_hi > kblocks) kb_hi = kblocks;
  const int k_len = kb_per_split * 64;
  const uint8_t* q = qblocks + (static_cast<size_t>(g) * kblocks + kb_lo) * 4096 + tid * 16;
  const uint8_t* sz = szblocks + static_cast<size_t>(g) * q_groups * 384;
  constexpr int UNR = 4;                      // K blocks whose loads travel together
  uint4 w[UNR][2];
  skptx::griddep_wait();
#pragma unroll
  for (int u = 0; u < UNR; ++u) {
    const int kk = kb_lo + u < kb_hi ? u : 0;   // (past the range: a repeated load, not used)
    w[u][0] = ld_stream_v4(q + static_cast<size_t>(kk) * 4096);
    w[u][1] = ld_stream_v4(q + static_cast<size_t>(kk) * 4096 + 2048);
  }
  float inv[M];
  stage_activations_scaled<M>(sAh, s_max, A, lda, K, kb_lo * 64, k_len, tid, inv);
  // C[m][row] = sum over scale groups of s * sum over the group's K of (q - z) * a.  The inner
  // sum: exact integers (q - z) times fp16 activations, 16 terms at a time in fp16 (two chains of
  // eight fused multiply-adds on pairs), then in fp32; the scale once per group.  (The reference
  // accumulates in fp16 throughout, streamk_fp16_ladder_block_reduce_q4.py:25.)
  float acc[M], part[M];
#pragma unroll
  for (int m = 0; m < M; ++m) { acc[m] = 0.f; part[m] = 0.f; }
  int cur_blk = -1;
  float scale = 0.f;
  __half2 c0 = __float2half2_rn(1024.f), c1 = __float2half2_rn(-64.f);
  for (int kb = kb_lo; kb < kb_hi; kb += UNR) {
#pragma unroll
    for (int u = 0; u < UNR; ++u) {
      if (kb + u >= kb_hi) break;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int blk = (2 * (kb + u) + h) >> gshift;   // scale group of this 32-wide half step
        if (blk != cur_blk) {
#pragma unroll
          for (int m = 0; m < M; ++m) { acc[m] = fmaf(scale, part[m], acc[m]); part[m] = 0.f; }
          cur_blk = blk;
          const uint8_t* b = sz + static_cast<size_t>(blk) * 384;
          scale = __half2float(*reinterpret_cast<const __half*>(b + tid * 2));
          const float z = static_cast<float>(b[256 + tid]);
          c0 = __float2half2_rn(1024.f + z);
          c1 = __float2half2_rn(-(64.f + z));
        }
        const uint32_t words[4] = {w[u][h].x, w[u][h].y, w[u][h].z, w[u][h].w};
        const uint16_t* a0 = sAh + ((kb + u - kb_lo) * 64 + h * 32);
        __half2 p0[M], p1[M];
#pragma unroll
        for (int m = 0; m < M; ++m) { p0[m] = __float2half2_rn(0.f); p1[m] = p0[m]; }
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          __half2 d[4];
          nibbles8(words[c], c0, c1, d);
#pragma unroll
          for (int m = 0; m < M; ++m) {
            const uint4 x = *reinterpret_cast<const uint4*>(a0 + m * k_len + c * 8);   // (same address in every lane)
            const __half2* a = reinterpret_cast<const __half2*>(&x);
            p0[m] = __hfma2(d[0], a[0], p0[m]);
            p1[m] = __hfma2(d[1], a[1], p1[m]);
            p0[m] = __hfma2(d[2], a[2], p0[m]);
            p1[m] = __hfma2(d[3], a[3], p1[m]);
          }
        }
#pragma unroll
        for (int m = 0; m < M; ++m) {
          const float2 f = __half22float2(__hadd2(p0[m], p1[m]));
          part[m] += f.x + f.y;
        }
      }
    }
    q += static_cast<size_t>(UNR) * 4096;
    if (kb + UNR < kb_hi) {
#pragma unroll
      for (int u = 0; u < UNR; ++u) {
        const int kk = kb + UNR + u < kb_hi ? u : 0;
        w[u][0] = ld_stream_v4(q + static_cast<size_t>(kk) * 4096);
        w[u][1] = ld_stream_v4(q + static_cast<size_t>(kk) * 4096 + 2048);
      }
    }
  }
#pragma unroll
  for (int m = 0; m < M; ++m) sums[m * SK_GEMV_ROWS + tid] = fmaf(scale, part[m], acc[m]) * inv[m];
  skptx::griddep_launch_dependents();
  __syncthreads();
  finish_group<M>(sums, parts, counters, C, ldc, N, g, s, S, 0, tid, GEMV_THREADS_Q4, &s_last);
}

}  // namespace

// Launchers, called by sk_gemm_f16 / sk_gemm_w4a16 once the schedule has resolved to
// SK_SCHED_GEMV (their argument checks have run).  ws: carved workspace of the device.
int sk_launch_gemv_f16(const sk_problem* prob, const void* A, const void* B, void* C, const SkWorkspace& ws,
                       int num_sms, int dev_sms, void* stream) {
  SkGemvPlan pl;
  if (prob->layout != SK_LAYOUT_NT) return SK_ERR_ARG;
  if (!sk_gemv_plan(1, prob->M, prob->N, prob->K, num_sms, &pl)) return SK_ERR_SHAPE;
  if (pl.groups > 4 * dev_sms) return SK_ERR_LIMIT;
  if ((prob->K & 7) != 0 || (prob->lda & 7) != 0 || (prob->ldb & 7) != 0) return SK_ERR_ALIGN;
  const bool bf16 = (prob->flags & SK_FLAG_BF16) != 0;
  const bool pdl = (prob->flags & SK_FLAG_PDL) != 0;
  const size_t smem = static_cast<size_t>(prob->M) * pl.k_per_split * sizeof(float);
  const cudaStream_t cs = static_cast<cudaStream_t>(stream);
  const uint16_t* a = static_cast<const uint16_t*>(A);
  const uint16_t* b = static_cast<const uint16_t*>(B);
  uint16_t* c = static_cast<uint16_t*>(C);
  cudaError_t e = cudaSuccess;
#define SK_GEMV_F16(MM, BB)                                                                              \
  e = sk_launch(sk_gemv_f16_kernel<MM, BB>, pl.grid, GEMV_THREADS_F16, smem, cs, 1, pdl, a, prob->lda, b, \
                prob->ldb, c, prob->ldc, prob->N, prob->K, pl.k_per_split, pl.splits, ws.part_slots, ws.counters)
  switch (prob->M * 2 + (bf16 ? 1 : 0)) {
    case 2: SK_GEMV_F16(1, false); break;
    case 3: SK_GEMV_F16(1, true); break;
    case 4: SK_GEMV_F16(2, false); break;
    case 5: SK_GEMV_F16(2, true); break;
    case 6: SK_GEMV_F16(3, false); break;
    case 7: SK_GEMV_F16(3, true); break;
    case 8: SK_GEMV_F16(4, false); break;
    case 9: SK_GEMV_F16(4, true); break;
    default: return SK_ERR_SHAPE;
  }
#undef SK_GEMV_F16
  if (e != cudaSuccess) return sk_set_cuda_error(e);
  return SK_OK;
}

int sk_launch_gemv_q4(const sk_problem* prob, const void* A, const void* qblocks, const void* szblocks, void* C,
                      int gshift, int q_groups, const SkWorkspace& ws, int num_sms, int dev_sms, void* stream) {
  SkGemvPlan pl;
  if (!sk_gemv_plan(2, prob->M, prob->N, prob->K, num_sms, &pl)) return SK_ERR_SHAPE;
  if (pl.groups > 4 * dev_sms) return SK_ERR_LIMIT;
  if ((prob->flags & SK_FLAG_BF16) != 0) return SK_ERR_ARG;
  const bool pdl = (prob->flags & SK_FLAG_PDL) != 0;
  const int kblocks = prob->K / 64, kb_per_split = pl.k_per_split / 64;
  const size_t smem = static_cast<size_t>(prob->M) * pl.k_per_split * sizeof(uint16_t);
  const cudaStream_t cs = static_cast<cudaStream_t>(stream);
  const uint16_t* a = static_cast<const uint16_t*>(A);
  const uint8_t* qb = static_cast<const uint8_t*>(qblocks);
  const uint8_t* sz = static_cast<const uint8_t*>(szblocks);
  uint16_t* c = static_cast<uint16_t*>(C);
  cudaError_t e = cudaSuccess;
#define SK_GEMV_Q4(MM)                                                                                 \
  e = sk_launch(sk_gemv_q4_kernel<MM>, pl.grid, GEMV_THREADS_Q4, smem, cs, 1, pdl, a, prob->lda, qb, sz, c, \
                prob->ldc, prob->N, prob->K, kblocks, kb_per_split, pl.splits, gshift, q_groups,       \
                ws.part_slots, ws.counters)
  switch (prob->M) {
    case 1: SK_GEMV_Q4(1); break;
    case 2: SK_GEMV_Q4(2); break;
    case 3: SK_GEMV_Q4(3); break;
    case 4: SK_GEMV_Q4(4); break;
    default: return SK_ERR_SHAPE;
  }
#undef SK_GEMV_Q4
  if (e != cudaSuccess) return sk_set_cuda_error(e);
  return SK_OK;
}
