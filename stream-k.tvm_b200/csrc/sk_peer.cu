// Device memory shared between the processes of one machine (one process per GPU), for the
// result matrices the fused all-gather (sk_gemm_f16_gather) writes into: allocate + export on
// the owner, map on the peers.  CUDA IPC handles are plain bytes; how they travel between the
// processes is the caller's business (torch.distributed object collectives in the Python
// layer).  No counterpart in the reference, which is a single-GPU study.
#include "sk_common.cuh"

static_assert(sizeof(cudaIpcMemHandle_t) == SK_PEER_HANDLE_BYTES, "handle size is part of the ABI");

extern "C" int sk_peer_alloc(size_t bytes, void** ptr, void* handle) {
  if (!ptr || !handle || bytes == 0) return SK_ERR_ARG;
  void* d = nullptr;
  cudaError_t e = cudaMalloc(&d, bytes);
  if (e != cudaSuccess) return sk_set_cuda_error(e);
  cudaIpcMemHandle_t h;
  e = cudaIpcGetMemHandle(&h, d);
  if (e != cudaSuccess) {
    cudaFree(d);
    return sk_set_cuda_error(e);
  }
  memcpy(handle, &h, sizeof(h));
  *ptr = d;
  return SK_OK;
}

extern "C" int sk_peer_open(const void* handle, void** ptr) {
  if (!handle || !ptr) return SK_ERR_ARG;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  void* d = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&d, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return sk_set_cuda_error(e);
  *ptr = d;
  return SK_OK;
}

extern "C" int sk_peer_close(void* ptr) {
  if (!ptr) return SK_ERR_ARG;
  cudaError_t e = cudaIpcCloseMemHandle(ptr);
  if (e != cudaSuccess) return sk_set_cuda_error(e);
  return SK_OK;
}

extern "C" int sk_peer_free(void* ptr) {
  if (!ptr) return SK_ERR_ARG;
  cudaError_t e = cudaFree(ptr);
  if (e != cudaSuccess) return sk_set_cuda_error(e);
  return SK_OK;
}

// ---------------------------------------------------------------------------------------
// Second half of the fused reduce-scatter (sk_gemm_f16_scatter): the receive buffer of a GPU
// holds n_parts fp32 partial sums [M, Nb] of its column block, one per sender; they are added in
// ascending sender order (so the result is bitwise reproducible) and rounded once to the 16-bit
// result type.  HBM-bound: (4 n_parts + 2) bytes per element, one float4 per thread and part.
// ---------------------------------------------------------------------------------------
namespace {
__global__ void reduce_partials_kernel(const float4* __restrict__ parts, int n_parts, size_t quads_per_part,
                                       int quads_per_row, uint2* __restrict__ C, int ldc_quads, int bf16) {
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < quads_per_part; i += stride) {
    float4 acc = __ldcs(parts + i);
    for (int g = 1; g < n_parts; ++g) {
      const float4 x = __ldcs(parts + static_cast<size_t>(g) * quads_per_part + i);
      acc.x += x.x; acc.y += x.y; acc.z += x.z; acc.w += x.w;
    }
    uint2 o;
    if (bf16) {
      asm("cvt.rn.bf16x2.f32 %0, %2, %1;" : "=r"(o.x) : "f"(acc.x), "f"(acc.y));
      asm("cvt.rn.bf16x2.f32 %0, %2, %1;" : "=r"(o.y) : "f"(acc.z), "f"(acc.w));
    } else {
      asm("cvt.rn.f16x2.f32 %0, %2, %1;" : "=r"(o.x) : "f"(acc.x), "f"(acc.y));
      asm("cvt.rn.f16x2.f32 %0, %2, %1;" : "=r"(o.y) : "f"(acc.z), "f"(acc.w));
    }
    const size_t row = i / quads_per_row, q = i - row * quads_per_row;
    C[row * ldc_quads + q] = o;
  }
}
}  // namespace

extern "C" int sk_reduce_partials(const void* parts, int n_parts, int M, int Nb, void* C, int ldc, int flags,
                                  void* stream) {
  if (!parts || !C || n_parts < 1) return SK_ERR_ARG;
  if (M <= 0 || Nb <= 0 || (Nb & 3) != 0 || ldc < Nb || (ldc & 3) != 0) return SK_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(parts) & 15u) || (reinterpret_cast<uintptr_t>(C) & 7u)) return SK_ERR_ALIGN;
  const size_t quads = static_cast<size_t>(M) * (Nb / 4);
  const int grid = static_cast<int>((quads + 255) / 256 < 148 * 8 ? (quads + 255) / 256 : 148 * 8);
  reduce_partials_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const float4*>(parts), n_parts, quads, Nb / 4, static_cast<uint2*>(C), ldc / 4,
      (flags & SK_FLAG_BF16) ? 1 : 0);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return sk_set_cuda_error(e);
  return SK_OK;
}
