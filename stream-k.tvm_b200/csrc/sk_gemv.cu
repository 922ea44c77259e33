// Small-M path (SK_SCHED_GEMV): C[M,N] = A[M,K] . W^T for a few rows of activations.
//
// With a few rows of activations a weight is used only a few times, the product is a stream of
// the weight matrix, and the tensor-memory kernels spend more time on their fixed costs
// (tensor-memory allocation, mbarrier rings, a cluster exchange or a workspace fix-up: 6-8 us per
// launch) than the stream itself takes.  These kernels have none of that: many small CTAs, loads
// kept in flight per thread or per warp, and partial sums that meet in shared memory (W4A16: the
// K slices of a CTA's warps) or in the workspace (a split of K across CTAs, added in split order
// by the last CTA of a row group to arrive: a counter tells), always in a fixed order, so the
// result is bitwise reproducible like the block-reduce fixup's.  The reference has no such path:
// its kernels are tiled for the tensor cores at every M (streamk_fp16.py:143-371,
// streamk_fp16_ladder_block_reduce_q4.py:143-522).
//
// Three kernels:
//   fp16 / bf16 weights [N, K] row-major, M <= 4 (CUDA cores).  CTA (g, s) walks K range s of
//     the 128 rows of group g; a warp takes 16 rows, eight at a time; its 32 lanes read 512
//     contiguous bytes of one row per instruction (8 K values each), the activations of the
//     lane's K values sit in registers for all eight rows, and the lanes' sums meet in a
//     shuffle tree at the end.
//   W4A16 packed image (sk_prepack_q4: [row block][K block] of [half][row][16 B]) with scale
//     groups of 32 or 64, M <= 4 (CUDA cores).  A CTA takes 32 rows, a warp a slice of K, a
//     thread one weight row: it reads its 2 x 16 bytes of a K block (a warp: 512 contiguous
//     bytes each), turns the nibbles into fp16 pairs (q - z) with one logic and one arithmetic
//     instruction per pair, multiplies with activations that every lane reads from the same
//     shared-memory address (16 terms at a time in fp16, then fp32), and applies the scale once
//     per scale group.
//   W4A16 with scale groups of 128 and more, M <= 16 (register-level tensor-core instructions
//     on nibbles read as fp16 subnormals; described at the kernel).
#include "sk_common.cuh"

namespace {

constexpr int GEMV_THREADS_F16 = 256;
constexpr int GEMV_THREADS_Q4 = 32 * SK_GEMV_Q4_WARPS;   // at most

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

// Partial sums of CTA (g, s) are at parts[((g * S + s) * M + m) * rows + row]; the last CTA of
// group g to arrive adds them over s = 0 .. S-1 in that order and stores C[m][g * rows + row].
__device__ __forceinline__ void finish_group(const float* sums /* shared: [M][rows] */, int M, int rows, float* parts,
                                             uint32_t* counters, uint16_t* C, int ldc, int N, int g, int s,
                                             int S, int bf16, int tid, int nthreads, uint32_t* s_last) {
  const int row0 = g * rows, items = M * rows;
  if (S == 1) {
    for (int i = tid; i < items; i += nthreads) {
      const int m = i / rows, r = i - m * rows;
      if (row0 + r < N) C[static_cast<size_t>(m) * ldc + row0 + r] = static_cast<uint16_t>(pack_out(sums[i], bf16));
    }
    return;
  }
  float* mine = parts + static_cast<size_t>(g * S + s) * items;
  for (int i = tid; i < items; i += nthreads) __stcg(mine + i, sums[i]);
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const uint32_t old = atomicAdd(counters + g, 1u);
    *s_last = old == static_cast<uint32_t>(S - 1) ? 1u : 0u;
  }
  __syncthreads();
  if (*s_last == 0u) return;
  __threadfence();
  const float* all = parts + static_cast<size_t>(g * S) * items;
  for (int i = tid; i < items; i += nthreads) {
    const int m = i / rows, r = i - m * rows;
    float acc = 0.f;
    for (int j0 = 0; j0 < S; j0 += 8) {     // eight loads in flight, added in split order
      float v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u)
        v[u] = __ldcg(all + static_cast<size_t>(j0 + u < S ? j0 + u : S - 1) * items + i);
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
__global__ void __launch_bounds__(GEMV_THREADS_F16, M == 1 ? 4 : 1)
sk_gemv_f16_kernel(const uint16_t* __restrict__ A, int lda, const uint16_t* __restrict__ B, int ldb,
                   uint16_t* __restrict__ C, int ldc, int N, int K, int k_per_split, int S, float* parts,
                   uint32_t* counters) {
  extern __shared__ __align__(16) float sA[];   // [M][k_per_split]
  __shared__ float sums[M * SK_GEMV_ROWS];
  __shared__ uint32_t s_last;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = blockIdx.x / S, s = blockIdx.x - g * S;
  const int k_lo = s * k_per_split;
  int k_hi = k_lo + k_per_split;
  if (k_hi > K) k_hi = K;
  uint4 w[8];
  auto load = [&](int r0, int k) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      // (rows past N repeat the last row: loaded, never stored)
      const int r = r0 + j < N ? r0 + j : N - 1;
      w[j] = ld_stream_v4(B + static_cast<size_t>(r) * ldb + k);
    }
  };
  skptx::griddep_wait();
  // the first eight loads travel while the activations are staged
  const bool first = k_lo + lane * 8 < k_hi;
  if (first) load(g * SK_GEMV_ROWS + warp * 16, k_lo + lane * 8);
  stage_activations<M, BF16>(sA, A, lda, K, k_lo, k_per_split, tid, GEMV_THREADS_F16);
  __syncthreads();
#pragma unroll 1
  for (int batch = 0; batch < 2; ++batch) {
    const int r0 = g * SK_GEMV_ROWS + warp * 16 + batch * 8;
    float acc[8][M];
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int m = 0; m < M; ++m) acc[j][m] = 0.f;
    for (int k = k_lo + lane * 8; k < k_hi; k += 256) {
      if (batch != 0 || k != k_lo + lane * 8) load(r0, k);
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
  finish_group(sums, M, SK_GEMV_ROWS, parts, counters, C, ldc, N, g, s, S, BF16 ? 1 : 0, tid, GEMV_THREADS_F16, &s_last);
}

// ------------------------------------------------------------------------------------ W4A16
// A warp's slice of the activations as fp16 in its own piece of shared memory, sA[m][k - k_lo],
// each row multiplied by a power of two that brings the slice's largest magnitude into
// [32, 64): the inner sums below are taken in fp16 over 16 terms of |q - z| <= 15, which then
// stay below 16 * 15 * 64 whatever the activations are (an outlier of a few thousand would
// overflow them otherwise).  inv[m] undoes the factor (exactly) on the fp32 side.  Warp-local:
// no CTA-wide barrier.
template <int M>
__device__ __forceinline__ void stage_slice_scaled(uint16_t* sA, const uint16_t* A, int lda, int k_lo, int k_len,
                                                   int k_stride, int lane, float (&inv)[M]) {
  const int chunks = k_len >> 3;   // 16-byte chunks per row
#pragma unroll
  for (int m = 0; m < M; ++m) {
    __half2 mx = __float2half2_rn(0.f);
    for (int c = lane; c < chunks; c += 32) {
      const uint4 v = *reinterpret_cast<const uint4*>(A + static_cast<size_t>(m) * lda + k_lo + c * 8);
      *reinterpret_cast<uint4*>(sA + m * k_stride + c * 8) = v;
      const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
      for (int e = 0; e < 4; ++e) mx = __hmax2(mx, __habs2(h[e]));
    }
    float f = fmaxf(__low2float(mx), __high2float(mx));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) f = fmaxf(f, __shfl_xor_sync(0xffffffffu, f, o));
    int e = 132 - static_cast<int>((__float_as_uint(f) >> 23) & 0xFFu);   // 2^e * max in [32, 64)
    e = e < -11 ? -11 : (e > 14 ? 14 : e);                                 // 2^e is a normal fp16
    const __half2 up = __float2half2_rn(__uint_as_float(static_cast<uint32_t>(127 + e) << 23));
    inv[m] = __uint_as_float(static_cast<uint32_t>(127 - e) << 23);
    for (int c = lane; c < chunks; c += 32) {   // (the chunks this lane wrote)
      uint4* dst = reinterpret_cast<uint4*>(sA + m * k_stride + c * 8);
      uint4 v = *dst;
      __half2* h = reinterpret_cast<__half2*>(&v);
#pragma unroll
      for (int q = 0; q < 4; ++q) h[q] = __hmul2(h[q], up);
      *dst = v;
    }
  }
  __syncwarp();
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

constexpr int Q4_UNR = 2;   // K blocks (64 of K each) whose loads travel together: four 16-byte loads per thread

// The packed words of up to Q4_UNR K blocks of this thread's row (`left` = K blocks that remain;
// past them a repeated load, not used).
__device__ __forceinline__ void q4_load(uint4 (&w)[Q4_UNR][2], const uint8_t* q, int left) {
#pragma unroll
  for (int u = 0; u < Q4_UNR; ++u) {
    const uint8_t* src = q + static_cast<size_t>(u < left ? u : 0) * 4096;
    w[u][0] = ld_stream_v4(src);
    w[u][1] = ld_stream_v4(src + 2048);
  }
}

// C[m][row] = sum over scale groups of s * sum over the group's K of (q - z) * a.  The inner sum:
// exact integers (q - z) times fp16 activations, 16 terms at a time in fp16 (two chains of eight
// fused multiply-adds on pairs), then in fp32; the scale once per group.  (The reference
// accumulates in fp16 throughout, streamk_fp16_ladder_block_reduce_q4.py:25.)
template <int M>
struct Q4Sum {
  float acc[M], part[M], scale;
  __half2 c0, c1;
  int cur_blk;
};

// One step: K blocks kb .. kb + Q4_UNR - 1 (below kb_hi) of the thread's row against the
// activations at `a` (shared memory, rows k_stride apart).  sz: the row's scale of group 0.
template <int M>
__device__ __forceinline__ void q4_step(Q4Sum<M>& t, const uint4 (&w)[Q4_UNR][2], int kb, int kb_hi,
                                        const uint8_t* sz, int rb, int gshift, const uint16_t* a,
                                        int k_stride) {
#pragma unroll
  for (int u = 0; u < Q4_UNR; ++u) {
    if (kb + u >= kb_hi) break;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int blk = (2 * (kb + u) + h) >> gshift;   // scale group of this 32-wide half step
      if (blk != t.cur_blk) {
#pragma unroll
        for (int m = 0; m < M; ++m) { t.acc[m] = fmaf(t.scale, t.part[m], t.acc[m]); t.part[m] = 0.f; }
        t.cur_blk = blk;
        const uint8_t* b = sz + static_cast<size_t>(blk) * 384;
        t.scale = __half2float(*reinterpret_cast<const __half*>(b));
        const float z = static_cast<float>(b[256 - rb]);   // (b points rb * 2 into the scales: 256 + rb from their start)
        t.c0 = __float2half2_rn(1024.f + z);
        t.c1 = __float2half2_rn(-(64.f + z));
      }
      const uint32_t words[4] = {w[u][h].x, w[u][h].y, w[u][h].z, w[u][h].w};
      const uint16_t* a0 = a + (u * 64 + h * 32);
      __half2 p0[M], p1[M];
#pragma unroll
      for (int m = 0; m < M; ++m) { p0[m] = __float2half2_rn(0.f); p1[m] = p0[m]; }
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        __half2 d[4];
        nibbles8(words[c], t.c0, t.c1, d);
#pragma unroll
        for (int m = 0; m < M; ++m) {
          const uint4 x = *reinterpret_cast<const uint4*>(a0 + m * k_stride + c * 8);   // (same address in every lane)
          const __half2* av = reinterpret_cast<const __half2*>(&x);
          p0[m] = __hfma2(d[0], av[0], p0[m]);
          p1[m] = __hfma2(d[1], av[1], p1[m]);
          p0[m] = __hfma2(d[2], av[2], p0[m]);
          p1[m] = __hfma2(d[3], av[3], p1[m]);
        }
      }
#pragma unroll
      for (int m = 0; m < M; ++m) {
        const float2 f = __half22float2(__hadd2(p0[m], p1[m]));
        t.part[m] += f.x + f.y;
      }
    }
  }
}

// CTA (g, s): 32 weight rows times `slices` pieces of the CTA's K range, one per warp.  A thread
// owns one weight row over its warp's K slice, two K blocks (128 of K) per step, the next step's
// loads in flight while it sums (the first step's while the warp stages its activations).  The
// slices' sums meet in shared memory and are added in slice order.
template <int M>
__global__ void __launch_bounds__(GEMV_THREADS_Q4)
sk_gemv_q4_kernel(const uint16_t* __restrict__ A, int lda, const uint8_t* __restrict__ qblocks,
                  const uint8_t* __restrict__ szblocks, uint16_t* __restrict__ C, int ldc, int N, int K,
                  int kblocks, int kb_per_split, int kb_per_slice, int S, int gshift, int q_groups,
                  float* parts, uint32_t* counters) {
  extern __shared__ __align__(16) uint16_t sAh[];   // [warp][M][kb_per_slice * 64]
  __shared__ float red[M * GEMV_THREADS_Q4];        // [slice][m][row of the CTA]
  __shared__ float sums[M * 32];
  __shared__ uint32_t s_last;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int nthreads = blockDim.x, slices = nthreads >> 5;
  const int g = blockIdx.x / S, s = blockIdx.x - g * S;
  const int row = g * 32 + lane;                        // weight row of this thread
  const int rb = row & 127;                             // ... inside its 128-row block
  int kb_end = (s + 1) * kb_per_split;
  if (kb_end > kblocks) kb_end = kblocks;
  const int kb_lo = s * kb_per_split + warp * kb_per_slice;
  int kb_hi = kb_lo + kb_per_slice;
  if (kb_hi > kb_end) kb_hi = kb_end;
  const int k_slice = kb_per_slice * 64;
  const uint8_t* q = qblocks + (static_cast<size_t>(row >> 7) * kblocks + kb_lo) * 4096 + rb * 16;
  const uint8_t* sz = szblocks + static_cast<size_t>(row >> 7) * q_groups * 384;
  uint16_t* sA = sAh + static_cast<size_t>(warp) * M * k_slice;
  float inv[M];
  Q4Sum<M> sum;
#pragma unroll
  for (int m = 0; m < M; ++m) { sum.acc[m] = 0.f; sum.part[m] = 0.f; inv[m] = 0.f; }
  sum.scale = 0.f;
  sum.cur_blk = -1;
  sum.c0 = __float2half2_rn(1024.f);
  sum.c1 = __float2half2_rn(-64.f);
  skptx::griddep_wait();
  if (kb_lo < kb_hi) {
    // Two sets of registers: the loads of one step travel while the other is summed.
    uint4 w0[Q4_UNR][2], w1[Q4_UNR][2];
    q4_load(w0, q, kb_hi - kb_lo);
    stage_slice_scaled<M>(sA, A, lda, kb_lo * 64, (kb_hi - kb_lo) * 64, k_slice, lane, inv);
    sz += rb * 2;
    for (int kb = kb_lo; kb < kb_hi; kb += 2 * Q4_UNR) {
      if (kb + Q4_UNR < kb_hi) q4_load(w1, q + static_cast<size_t>(Q4_UNR) * 4096, kb_hi - kb - Q4_UNR);
      q4_step<M>(sum, w0, kb, kb_hi, sz, rb, gshift, sA + (kb - kb_lo) * 64, k_slice);
      if (kb + Q4_UNR >= kb_hi) break;
      q += static_cast<size_t>(2 * Q4_UNR) * 4096;
      if (kb + 2 * Q4_UNR < kb_hi) q4_load(w0, q, kb_hi - kb - 2 * Q4_UNR);
      q4_step<M>(sum, w1, kb + Q4_UNR, kb_hi, sz, rb, gshift, sA + (kb + Q4_UNR - kb_lo) * 64, k_slice);
    }
  }
#pragma unroll
  for (int m = 0; m < M; ++m) red[(warp * M + m) * 32 + lane] = fmaf(sum.scale, sum.part[m], sum.acc[m]) * inv[m];
  skptx::griddep_launch_dependents();
  __syncthreads();
  for (int i = tid; i < M * 32; i += nthreads) {
    float v = red[i];                           // slice 0 of (m, row) = i
    for (int j = 1; j < slices; ++j) v += red[j * M * 32 + i];
    sums[i] = v;
  }
  __syncthreads();
  finish_group(sums, M, 32, parts, counters, C, ldc, N, g, s, S, 0, tid, nthreads, &s_last);
}

// --------------------------------------------------------- W4A16, scale groups of 128 and more
// The same split of the work (32 weight rows per CTA, one K slice per warp), with the products
// on the tensor cores through register-level mma.sync (m16n8k16, fp32 accumulators): the eight
// columns of the instruction hold the rows of activations, so up to eight cost what one costs
// (nine to sixteen: a second column tile, twice the instructions).
//
// No arithmetic is spent on turning nibbles into numbers: a nibble masked into bits 0-3 of an
// fp16 is the subnormal q * 2^-24, which the tensor cores multiply exactly; fp32 accumulators
// take it from there, so the activations go in as they are, whatever their range.  A second
// set of accumulators takes the activations against a tile of ones: the sum that the
// zero-point multiplies.  Scales and zero-points are applied to the accumulators once per step
// of 128 along K, which is why the scale group must be a multiple of 128:
//   C[m][row] += s * (sum q a  -  z * sum a).
//
// Operand layout.  Lane (g = lane / 4, t = lane % 4) holds, of a step, the 16 bytes (32 values
// of K) of piece t (piece = K block t / 2, half t % 2) for weight rows g, g + 8, g + 16, g + 24
// of the CTA's 32: rows g, g + 8 are rows g, g + 8 of the first 16-row operand tile, the other
// two of the second.  A packed word holds 8 consecutive K values, the even ones in its low
// half: the mask 0x000F000F leaves values 0, 1 of the eight as a pair, the same mask after a
// shift by 8 values 4, 5, and these four are the lane's K slots of one instruction; shifts by
// 4 and 12 give 2, 3 and 6, 7 for the next.  The activations' 16 bytes for the same eight K
// values (straight from global memory through L1, row g of A for the lane) hold the pairs
// (0,1) (2,3) (4,5) (6,7): first and third word for the one, second and fourth for the other.
__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
               "{%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ld_cached_v4(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

// The weights reach the lanes through a ring of Q4M_DEPTH steps per warp in shared memory,
// filled by asynchronous copies.  Two reasons: the bytes in flight cost no registers, and the
// copies can be issued the way the memory pipeline likes them (lane = row: a warp-wide copy is
// 512 contiguous bytes), whereas the instruction's operand layout, read from global memory
// directly, makes every quarter-warp touch four different lines (measured: the L1 data pipe
// at 70 % of its wavefront rate with HBM at 35 %).  A slot holds the step's four pieces of
// 32 rows x 16 bytes, 544 bytes apart so that the four pieces a quarter-warp reads fall on
// different banks.  The rows' scales and zero-points of the step's group travel with them (a
// step ahead they would arrive a step late: every step of 128 has a group of its own).
constexpr int Q4M_DEPTH = 4;
constexpr int Q4M_PIECE = 544;
constexpr int Q4M_SZ = 4 * Q4M_PIECE;        // then the 32 rows' scales (64 bytes) and zero-points (32) of the step's group
constexpr int Q4M_SLOT = Q4M_SZ + 96;

__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ uint4 lds_v4(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}

// One warp, 32 weight rows from row0 on, `nsteps` steps of 128 along K from K block kb_lo on:
// acc[n][j][e] += the products of row row0 + 8 j + lane / 4 with row 8 n + 2 (lane % 4) + e of
// the activations.  ring_s: the warp's ring (shared-memory address); on return it is free again.
// NT: column tiles of the instruction (8 rows of activations each): M <= 8 NT.
template <int NT>
__device__ __forceinline__ void q4m_segment(float (&acc)[NT][4][2], const uint16_t* __restrict__ A, int lda, int M,
                                            const uint8_t* __restrict__ qblocks, const uint8_t* __restrict__ szblocks,
                                            int kblocks, int gshift, int q_groups, int row0, int kb_lo, int nsteps,
                                            uint32_t ring_s, int lane) {
  const int g8 = lane >> 2, t = lane & 3;
  const int rb0 = row0 & 127;                           // first row inside its 128-row block
  // copies: lane = row, piece p of step i = K block 2 i + p / 2, half p % 2
  const uint8_t* q = qblocks + (static_cast<size_t>(row0 >> 7) * kblocks + kb_lo) * 4096 + (rb0 + lane) * 16;
  // (a group's block: 128 scales, then 128 zero-points; lanes 0-3 copy the 32 rows' 64 bytes of
  // scales, lanes 4-5 their 32 bytes of zero-points)
  const uint8_t* sz = szblocks + static_cast<size_t>(row0 >> 7) * q_groups * 384 +
                      (lane < 4 ? rb0 * 2 + lane * 16 : 256 + rb0 + (lane - 4) * 16);
  auto issue = [&](int i) {   // step i of the segment into slot i % Q4M_DEPTH
    const uint8_t* src = q + static_cast<size_t>(i) * (2 * 4096);
    const uint32_t dst = ring_s + (i & (Q4M_DEPTH - 1)) * Q4M_SLOT + lane * 16;
#pragma unroll
    for (int p = 0; p < 4; ++p) cp_async_16(dst + p * Q4M_PIECE, src + p * 2048);
    if (lane < 6)
      cp_async_16(dst + Q4M_SZ, sz + static_cast<size_t>((2 * (kb_lo + 2 * i)) >> gshift) * 384);   // (dst: lane * 16 into the tail)
  };
#pragma unroll
  for (int d = 0; d < Q4M_DEPTH; ++d) {
    if (d < nsteps) issue(d);
    cp_async_commit();
  }
  // the activations this lane feeds: rows g, 8 + g of A (column g of the operand's tiles; past
  // M: the last row, into columns that nobody reads), piece t of the step
  const uint16_t* aB[NT];
#pragma unroll
  for (int n = 0; n < NT; ++n)
    aB[n] = A + static_cast<size_t>(8 * n + g8 < M ? 8 * n + g8 : M - 1) * lda + kb_lo * 64 + t * 32;
  const uint32_t frag_s = ring_s + t * Q4M_PIECE + g8 * 16;   // piece t, rows g + 8 j
  for (int i = 0; i < nsteps; ++i) {
    const uint32_t slot = (i & (Q4M_DEPTH - 1)) * Q4M_SLOT;
    uint4 x[NT][4];   // the step's activations (L1: every CTA of the SM reads the same few KB)
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
      for (int cw = 0; cw < 4; ++cw) x[n][cw] = ld_cached_v4(aB[n] + i * 128 + cw * 8);
    cp_async_wait<Q4M_DEPTH - 1>();   // all but the newest three groups: this lane's copies of step i have landed
    __syncwarp();                     // ... and every other lane's
    uint32_t wj[4][4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint4 v = lds_v4(frag_s + slot + j * 128);
      wj[j][0] = v.x; wj[j][1] = v.y; wj[j][2] = v.z; wj[j][3] = v.w;
    }
    // lane = row: its scale and zero-point
    uint16_t s_now;
    uint32_t z_now;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(s_now) : "r"(ring_s + slot + Q4M_SZ + lane * 2));
    asm volatile("ld.shared.u8 %0, [%1];" : "=r"(z_now) : "r"(ring_s + slot + Q4M_SZ + 64 + lane));
    __syncwarp();                     // the slot is read: refill it
    if (i + Q4M_DEPTH < nsteps) issue(i + Q4M_DEPTH);
    cp_async_commit();
    float c[NT][2][4], one[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) { c[n][0][e] = 0.f; c[n][1][e] = 0.f; one[n][e] = 0.f; }
    constexpr uint32_t ONES = 0x00010001u, NIB = 0x000F000Fu;   // 2^-24 twice; the low nibble of each half
#pragma unroll
    for (int cw = 0; cw < 4; ++cw) {
#pragma unroll
      for (int T = 0; T < 2; ++T) {
        const uint32_t wa = wj[2 * T][cw], wb = wj[2 * T + 1][cw];
        const uint32_t a0 = wa & NIB, a1 = wb & NIB, a2 = (wa >> 8) & NIB, a3 = (wb >> 8) & NIB;       // K values 0, 1, 4, 5
        const uint32_t b0 = (wa >> 4) & NIB, b1 = (wb >> 4) & NIB, b2 = (wa >> 12) & NIB, b3 = (wb >> 12) & NIB;   // 2, 3, 6, 7
#pragma unroll
        for (int n = 0; n < NT; ++n) {
          mma_16816(c[n][T], a0, a1, a2, a3, x[n][cw].x, x[n][cw].z);
          mma_16816(c[n][T], b0, b1, b2, b3, x[n][cw].y, x[n][cw].w);
        }
      }
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        mma_16816(one[n], ONES, ONES, ONES, ONES, x[n][cw].x, x[n][cw].z);
        mma_16816(one[n], ONES, ONES, ONES, ONES, x[n][cw].y, x[n][cw].w);
      }
    }
    // the scale and -z * scale of this lane's row (times the 2^24 of the subnormals) to the
    // lanes that hold the row's accumulators
    const float sc = __half2float(__ushort_as_half(s_now)) * 16777216.f;
    const float zs = -static_cast<float>(z_now) * sc;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float scj = __shfl_sync(0xffffffffu, sc, 8 * j + g8), zsj = __shfl_sync(0xffffffffu, zs, 8 * j + g8);
      const int T = j >> 1, e = (j & 1) * 2;
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        acc[n][j][0] = fmaf(c[n][T][e], scj, fmaf(zsj, one[n][0], acc[n][j][0]));
        acc[n][j][1] = fmaf(c[n][T][e + 1], scj, fmaf(zsj, one[n][1], acc[n][j][1]));
      }
    }
  }
  cp_async_wait<0>();
  __syncwarp();
}

// CTA (g, s): 32 weight rows, one K slice per warp (the split of the CUDA-core W4A16 kernel).
template <int NT>
__global__ void __launch_bounds__(GEMV_THREADS_Q4)
sk_gemv_q4_mma_kernel(const uint16_t* __restrict__ A, int lda, int M, const uint8_t* __restrict__ qblocks,
                      const uint8_t* __restrict__ szblocks, uint16_t* __restrict__ C, int ldc, int N, int K,
                      int kblocks, int kb_per_split, int kb_per_slice, int S, int gshift, int q_groups,
                      float* parts, uint32_t* counters) {
  extern __shared__ __align__(16) uint8_t ring[];    // [warp][Q4M_DEPTH][Q4M_SLOT], then red and sums
  __shared__ uint32_t s_last;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g8 = lane >> 2, t = lane & 3;
  const int nthreads = blockDim.x, slices = nthreads >> 5;
  float* red = reinterpret_cast<float*>(ring + slices * (Q4M_DEPTH * Q4M_SLOT));   // [slice][m][row of the CTA]
  float* sums = red + slices * M * 32;                                             // [m][row]
  const int g = blockIdx.x / S, s = blockIdx.x - g * S;
  int kb_end = (s + 1) * kb_per_split;
  if (kb_end > kblocks) kb_end = kblocks;
  const int kb_lo = s * kb_per_split + warp * kb_per_slice;
  int kb_hi = kb_lo + kb_per_slice;
  if (kb_hi > kb_end) kb_hi = kb_end;
  float acc[NT][4][2];
#pragma unroll
  for (int n = 0; n < NT; ++n)
#pragma unroll
    for (int j = 0; j < 4; ++j) { acc[n][j][0] = 0.f; acc[n][j][1] = 0.f; }
  skptx::griddep_wait();
  if (kb_lo < kb_hi)   // (K blocks come in pairs: K is a multiple of 128, and so is every slice)
    q4m_segment<NT>(acc, A, lda, M, qblocks, szblocks, kblocks, gshift, q_groups, g * 32, kb_lo, (kb_hi - kb_lo) >> 1,
                    static_cast<uint32_t>(__cvta_generic_to_shared(ring)) + warp * (Q4M_DEPTH * Q4M_SLOT), lane);
#pragma unroll
  for (int n = 0; n < NT; ++n)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int m = 8 * n + 2 * t + e;
        if (m < M) red[(warp * M + m) * 32 + 8 * j + g8] = acc[n][j][e];
      }
  skptx::griddep_launch_dependents();
  __syncthreads();
  for (int i = tid; i < M * 32; i += nthreads) {
    float v = red[i];                           // slice 0 of (m, row) = i
    for (int j = 1; j < slices; ++j) v += red[j * M * 32 + i];
    sums[i] = v;
  }
  __syncthreads();
  finish_group(sums, M, 32, parts, counters, C, ldc, N, g, s, S, 0, tid, nthreads, &s_last);
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
  const bool mma = gshift >= 2;   // scale groups of 128 and more: the tensor-core form
  if (!sk_gemv_plan(mma ? 2 : 3, prob->M, prob->N, prob->K, num_sms, &pl)) return SK_ERR_SHAPE;
  if (pl.splits > 1) {   // counters and partial sums of the workspace (P = dev_sms slots)
    if (pl.groups > 4 * dev_sms) return SK_ERR_LIMIT;
    const size_t need = static_cast<size_t>(pl.grid) * prob->M * pl.rows * sizeof(float);
    if (need > 2 * static_cast<size_t>(dev_sms) * SK_SLOT_BYTES) return SK_ERR_LIMIT;
  }
  if ((prob->flags & SK_FLAG_BF16) != 0) return SK_ERR_ARG;
  const bool pdl = (prob->flags & SK_FLAG_PDL) != 0;
  const int kblocks = prob->K / 64, kb_per_split = pl.k_per_split / 64, kb_per_slice = pl.k_per_slice / 64;
  const cudaStream_t cs = static_cast<cudaStream_t>(stream);
  const uint16_t* a = static_cast<const uint16_t*>(A);
  const uint8_t* qb = static_cast<const uint8_t*>(qblocks);
  const uint8_t* sz = static_cast<const uint8_t*>(szblocks);
  uint16_t* c = static_cast<uint16_t*>(C);
  cudaError_t e = cudaSuccess;
  if (mma) {
    // the rings of weights, then the slices' sums [slice][M][32] and their total [M][32]
    const size_t smem = static_cast<size_t>(pl.slices) * Q4M_DEPTH * Q4M_SLOT +
                        static_cast<size_t>(pl.slices + 1) * prob->M * 32 * sizeof(float);
    const size_t smem_max = static_cast<size_t>(SK_GEMV_Q4_WARPS) * Q4M_DEPTH * Q4M_SLOT +
                            static_cast<size_t>(SK_GEMV_Q4_WARPS + 1) * SK_GEMV_Q4_MAX_M * 32 * sizeof(float);
    if (prob->M <= 8) {
      if (smem > 40 * 1024)
        e = cudaFuncSetAttribute(sk_gemv_q4_mma_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_max);
      if (e == cudaSuccess)
        e = sk_launch(sk_gemv_q4_mma_kernel<1>, pl.grid, pl.threads, smem, cs, 1, pdl, a, prob->lda, prob->M, qb, sz,
                      c, prob->ldc, prob->N, prob->K, kblocks, kb_per_split, kb_per_slice, pl.splits, gshift,
                      q_groups, ws.part_slots, ws.counters);
    } else {
      if (smem > 40 * 1024)
        e = cudaFuncSetAttribute(sk_gemv_q4_mma_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_max);
      if (e == cudaSuccess)
        e = sk_launch(sk_gemv_q4_mma_kernel<2>, pl.grid, pl.threads, smem, cs, 1, pdl, a, prob->lda, prob->M, qb, sz,
                      c, prob->ldc, prob->N, prob->K, kblocks, kb_per_split, kb_per_slice, pl.splits, gshift,
                      q_groups, ws.part_slots, ws.counters);
    }
    if (e != cudaSuccess) return sk_set_cuda_error(e);
    return SK_OK;
  }
  const size_t smem = static_cast<size_t>(pl.slices) * prob->M * pl.k_per_slice * sizeof(uint16_t);
#define SK_GEMV_Q4(MM)                                                                                  \
  do {                                                                                                  \
    if (smem > 32 * 1024)                                                                               \
      e = cudaFuncSetAttribute(sk_gemv_q4_kernel<MM>, cudaFuncAttributeMaxDynamicSharedMemorySize,      \
                               SK_GEMV_Q4_SMEM_MAX);                                                    \
    if (e == cudaSuccess)                                                                               \
      e = sk_launch(sk_gemv_q4_kernel<MM>, pl.grid, pl.threads, smem, cs, 1, pdl, a, prob->lda, qb, sz, \
                    c, prob->ldc, prob->N, prob->K, kblocks, kb_per_split, kb_per_slice, pl.splits,     \
                    gshift, q_groups, ws.part_slots, ws.counters);                                      \
  } while (0)
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
