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
