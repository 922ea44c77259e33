// One-time weight re-layout kernels and the stand-alone int4 dequantiser.
//
// The reference prepares weights on the CPU with two third-party transforms:
// LadderPermutate regroups B[N,K] tile-major in register-fragment order
// (streamk_fp16_ladder.py:153,468-477) and LOP3Permutate interleaves nibbles so
// a lop3-based decode yields natural order (…_q4.py:568-595).  Their exact byte
// orders are private to those kernels' ldmatrix/mma.sync fragments, which do not
// exist on sm_100.  Here the pre-laid-out image is instead *the shared-memory
// image the UMMA descriptor reads*: blocks of 128 weight rows x 64 K-halves, each
// block stored exactly as a 128-byte-swizzled K-major tile, so the mainloop
// fetches a block with one 16 KB 1-D bulk copy and needs no tensor map.
#include "sk_common.cuh"

namespace {

// ---- fp16 "ladder" image -----------------------------------------------------
// Block (nb, kb) lives at ((nb * kblocks) + kb) * 16384 bytes.  Inside a block,
// row r (0..127), 16-byte chunk c (0..7) sits at r*128 + ((c ^ (r & 7)) * 16).
__global__ void prepack_ladder_kernel(const __half* __restrict__ B, int N, int K, int ldb,
                                      uint4* __restrict__ out, int nblocks, int kblocks,
                                      int vec_ok) {
  const size_t total = static_cast<size_t>(nblocks) * kblocks * 1024;  // 16-byte chunks
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t blk = i >> 10;
    const int in_blk = static_cast<int>(i & 1023);
    const int r = in_blk >> 3;
    const int c = (in_blk & 7) ^ (r & 7);   // i indexes the destination; recover the source chunk
    const int nb = static_cast<int>(blk / kblocks);
    const int kb = static_cast<int>(blk - static_cast<size_t>(nb) * kblocks);
    const int n = nb * 128 + r;
    const int k = kb * 64 + c * 8;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (n < N && k < K) {
      const __half* src = B + static_cast<size_t>(n) * ldb + k;
      if (vec_ok && k + 8 <= K) {
        v = *reinterpret_cast<const uint4*>(src);
      } else {
        __half h[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) h[e] = (k + e < K) ? src[e] : __float2half(0.f);
        v = *reinterpret_cast<uint4*>(h);
      }
    }
    out[i] = v;
  }
}

}  // namespace

extern "C" size_t sk_ladder_bytes(int N, int K) {
  if (N <= 0 || K <= 0) return 0;
  const size_t nb = (static_cast<size_t>(N) + 255) / 256 * 2;  // whole 256-row tiles
  const size_t kb = (static_cast<size_t>(K) + 63) / 64;
  return nb * kb * 16384;
}

extern "C" int sk_prepack_ladder(const void* B, int N, int K, int ldb, void* out, size_t out_bytes,
                                 void* stream) {
  if (!B || !out) return SK_ERR_ARG;
  if (N <= 0 || K <= 0 || ldb < K) return SK_ERR_SHAPE;
  if (out_bytes < sk_ladder_bytes(N, K)) return SK_ERR_WORKSPACE;
  if (reinterpret_cast<uintptr_t>(out) & 15u) return SK_ERR_ALIGN;
  const int nblocks = (N + 255) / 256 * 2;
  const int kblocks = (K + 63) / 64;
  const int vec_ok = ((reinterpret_cast<uintptr_t>(B) & 15u) == 0 && (ldb & 7) == 0) ? 1 : 0;
  const size_t total = static_cast<size_t>(nblocks) * kblocks * 1024;
  int grid = static_cast<int>((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  prepack_ladder_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __half*>(B), N, K, ldb, static_cast<uint4*>(out), nblocks, kblocks, vec_ok);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return sk_set_cuda_error(e);
  return SK_OK;
}
