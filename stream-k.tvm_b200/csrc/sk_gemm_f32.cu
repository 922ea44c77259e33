// fp32 Stream-K GEMM on CUDA cores (FFMA, no TF32): C = A . B (NN) or A . B^T (NT).
//
// Stands in for the TL kernel of streamk_fp32.py:57-177 (persistent grid, each
// CTA walks its share of tiles x K-iterations, partial tiles fixed up across
// CTAs).  Differences by design: the scheduler integers are kernel parameters
// (no recompilation per shape), C does not have to be pre-zeroed, partial sums
// meet in an fp32 workspace, and a deterministic fixup is available: the CTA that
// starts a split tile waits (with a time limit) for the partials of the CTAs that
// continue it and adds them in ascending CTA order.
#include "sk_common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, THREADS = 256;

template <bool B_IS_NT>
__global__ void __launch_bounds__(THREADS)
sk_gemm_f32_kernel(const float* __restrict__ A, const float* __restrict__ B, float* __restrict__ C,
                   SkParams p) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Bs[BK][BN + 4];
  __shared__ int s_last;

  const int tid = threadIdx.x;
  const int pid = blockIdx.x;
  const int ty = tid >> 4, tx = tid & 15;  // 16 x 16 threads, 4 x 4 outputs each
  const SkSched& s = p.sched;

  SkCursor cur;
  sk_cursor_init(s, pid, cur);
  SkSeg seg;
  while (sk_next(s, pid, cur, seg)) {
    int tm, tn;
    sk_tile_mn(s, seg.tile, tm, tn);
    const int m0 = tm * BM, n0 = tn * BN;

    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int kt = seg.k0; kt < seg.k1; ++kt) {
      const int kbase = kt * BK;
      // A tile: row (tid / 4), k quad (tid % 4)
      {
        const int r = tid >> 2, kq = (tid & 3) * 4;
        const int gm = m0 + r;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int gk = kbase + kq + e;
          As[kq + e][r] = (gm < p.M && gk < p.K) ? A[static_cast<size_t>(gm) * p.lda + gk] : 0.f;
        }
      }
      if (B_IS_NT) {
        const int r = tid >> 2, kq = (tid & 3) * 4;
        const int gn = n0 + r;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int gk = kbase + kq + e;
          Bs[kq + e][r] = (gn < p.N && gk < p.K) ? B[static_cast<size_t>(gn) * p.ldb + gk] : 0.f;
        }
      } else {
        const int kr = tid >> 4, nq = (tid & 15) * 4;
        const int gk = kbase + kr;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int gn = n0 + nq + e;
          Bs[kr][nq + e] = (gk < p.K && gn < p.N) ? B[static_cast<size_t>(gk) * p.ldb + gn] : 0.f;
        }
      }
      __syncthreads();
#pragma unroll
      for (int k = 0; k < BK; ++k) {
        float a[4], b[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
        for (int j = 0; j < 4; ++j) b[j] = Bs[k][tx * 4 + j];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
      }
      __syncthreads();
    }

    // ---------------------------------------------------------------- epilogue
    const bool whole = (seg.k0 == 0 && seg.k1 == s.iters_per_tile);
    const int row0 = m0 + ty * 4, col0 = n0 + tx * 4;
    auto store_c = [&](float (&v)[4][4]) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int gr = row0 + i;
        if (gr >= p.M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int gc = col0 + j;
          if (gc < p.N) C[static_cast<size_t>(gr) * p.ldc + gc] = v[i][j];
        }
      }
    };

    if (whole) {
      store_c(acc);
      continue;
    }
    int first, last;
    sk_tile_ctas(s, seg.tile, first, last);
    if (p.fixup == SK_FIXUP_ATOMIC) {
      float* slot = p.ws.acc_slots + static_cast<size_t>(first) * (SK_SLOT_BYTES / sizeof(float));
#pragma unroll
      for (int i = 0; i < 4; ++i)
        skptx::red_add_v4(slot + (ty * 4 + i) * BN + tx * 4, acc[i][0], acc[i][1], acc[i][2],
                          acc[i][3]);
      __threadfence();
      __syncthreads();
      if (tid == 0) {
        const uint32_t old = skptx::atom_add_acqrel_u32(p.ws.counters + first, 1u);
        s_last = (old == static_cast<uint32_t>(last - first)) ? 1 : 0;
      }
      __syncthreads();
      if (s_last) {
        __threadfence();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float4* q = reinterpret_cast<float4*>(slot + (ty * 4 + i) * BN + tx * 4);
          const float4 v = __ldcg(q);
          __stcg(q, make_float4(0.f, 0.f, 0.f, 0.f));
          acc[i][0] = v.x; acc[i][1] = v.y; acc[i][2] = v.z; acc[i][3] = v.w;
        }
        store_c(acc);
        if (tid == 0) p.ws.counters[first] = 0u;
      }
      __syncthreads();  // s_last is reused by the next segment
    } else {
      const size_t slot_f = SK_SLOT_FLOATS;
      if (seg.k0 != 0) {
        // peer: publish the partial, never wait
        float* slot = p.ws.part_slots + static_cast<size_t>(2 * pid) * slot_f;
#pragma unroll
        for (int i = 0; i < 4; ++i)
          __stcg(reinterpret_cast<float4*>(slot + (ty * 4 + i) * BN + tx * 4),
                 make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]));
        __threadfence();
        __syncthreads();
        if (tid == 0 && pid != p.drop_flag_cta) skptx::st_release_u32(p.ws.flag_head + pid, 1u);
      } else {
        // owner: add the peers' partials in ascending CTA order
        if (tid == 0) {
          int ok = 1;
          for (int peer = first + 1; peer <= last; ++peer) {
            if (!sk_wait_flag(p.ws.flag_head + peer, p.timeout_ns)) {
              sk_report(p.ws.status, SK_ERR_FIXUP_TIMEOUT, seg.tile, peer);
              ok = 0;
              break;
            }
          }
          s_last = ok;
        }
        __syncthreads();
        if (s_last) {
          for (int peer = first + 1; peer <= last; ++peer) {
            const float* slot = p.ws.part_slots + static_cast<size_t>(2 * peer) * slot_f;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float4 v =
                  __ldcg(reinterpret_cast<const float4*>(slot + (ty * 4 + i) * BN + tx * 4));
              acc[i][0] += v.x; acc[i][1] += v.y; acc[i][2] += v.z; acc[i][3] += v.w;
            }
          }
          store_c(acc);
        }
        __syncthreads();
        if (tid == 0 && s_last)
          for (int peer = first + 1; peer <= last; ++peer) p.ws.flag_head[peer] = 0u;
      }
    }
  }
}

}  // namespace

extern "C" int sk_gemm_f32(const sk_problem* prob, const float* A, const float* B, float* C,
                           void* ws, size_t ws_bytes, void* stream) {
  if (!prob || !A || !B || !C) return SK_ERR_ARG;
  if (prob->layout != SK_LAYOUT_NN && prob->layout != SK_LAYOUT_NT) return SK_ERR_ARG;
  if (prob->fixup != SK_FIXUP_ATOMIC && prob->fixup != SK_FIXUP_BLOCK_REDUCE) return SK_ERR_ARG;
  int num_sms = 0, dev_sms = 0;
  int st = sk_resolve_grid(prob, &num_sms, &dev_sms);
  if (st != SK_OK) return st;
  sk_problem resolved = *prob;   // SK_SCHED_AUTO -> a concrete schedule and tile
  sk_resolve_auto(&resolved, 0, num_sms);
  prob = &resolved;
  SkParams p;
  memset(&p, 0, sizeof(p));
  st = sk_make_sched(prob, 0, num_sms, nullptr, &p.sched, nullptr);
  if (st != SK_OK) return st;
  const bool nt = prob->layout == SK_LAYOUT_NT;
  if (prob->lda < prob->K || prob->ldc < prob->N || prob->ldb < (nt ? prob->K : prob->N))
    return SK_ERR_SHAPE;
  if (!ws || ws_bytes < sk_ws_total_bytes(dev_sms)) return SK_ERR_WORKSPACE;
  if ((reinterpret_cast<uintptr_t>(ws) & 255u) != 0) return SK_ERR_ALIGN;
  p.M = prob->M; p.N = prob->N; p.K = prob->K;
  p.lda = prob->lda; p.ldb = prob->ldb; p.ldc = prob->ldc;
  p.fixup = prob->fixup;
  p.drop_flag_cta = prob->test_drop_flag_cta - 1;
  p.timeout_ns = (prob->fixup_timeout_us > 0 ? static_cast<unsigned long long>(prob->fixup_timeout_us)
                                             : 2000000ULL) * 1000ULL;
  p.ws = sk_ws_carve(ws, dev_sms);  // layout fixed per device, whatever the grid
  cudaStream_t cs = static_cast<cudaStream_t>(stream);
  if (nt)
    sk_gemm_f32_kernel<true><<<p.sched.grid, THREADS, 0, cs>>>(A, B, C, p);
  else
    sk_gemm_f32_kernel<false><<<p.sched.grid, THREADS, 0, cs>>>(A, B, C, p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return sk_set_cuda_error(e);
  return SK_OK;
}

// ---------------------------------------------------------------------------------
// sk_gemm_f32_noalloc: the same kernel for callers that must not allocate.
//
// Some hosts of this library cannot provide a workspace: code running under a memory
// budget fixed at start-up, inside a region where cudaMalloc is forbidden (it
// synchronises the device and cannot appear during stream capture), or behind a plugin
// interface that hands over nothing but operand pointers.  For them the fixup scratch
// lives in the library image itself, in the array below.  It is sized for at most
// SK_NOALLOC_MAX_CTAS persistent CTAs, and every GPU that loads the library carries these
// ~6 MB until the process exits, whether or not this entry point is ever called.
// ---------------------------------------------------------------------------------
#include <mutex>

namespace {

constexpr int SK_NOALLOC_MAX_CTAS = 16;
constexpr size_t SK_NOALLOC_HEADER = 1024;   // status word, counters, done, flag_head, flag_tail
constexpr size_t SK_NOALLOC_BYTES =
    SK_NOALLOC_HEADER + 3 * static_cast<size_t>(SK_NOALLOC_MAX_CTAS) * SK_SLOT_BYTES;
static_assert(SK_WS_HEADER + 4 * sizeof(uint32_t) * SK_NOALLOC_MAX_CTAS <= SK_NOALLOC_HEADER,
              "header does not fit");

// In host code this name is only a handle for the runtime: it is not a device address and
// must never be passed to a kernel.  The address comes from cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_noalloc_scratch[SK_NOALLOC_BYTES];

std::mutex g_noalloc_mutex;
void* g_noalloc_ptr[64] = {nullptr};   // per device, filled on that device's first call

}  // namespace

extern "C" int sk_gemm_f32_noalloc(const sk_problem* prob, const float* A, const float* B, float* C,
                                   sk_status* host_status, void* stream) {
  if (!prob || !A || !B || !C) return SK_ERR_ARG;
  if (prob->layout != SK_LAYOUT_NN && prob->layout != SK_LAYOUT_NT) return SK_ERR_ARG;
  if (prob->fixup != SK_FIXUP_ATOMIC && prob->fixup != SK_FIXUP_BLOCK_REDUCE) return SK_ERR_ARG;
  // The scratch holds slots for SK_NOALLOC_MAX_CTAS CTAs: a larger grid is refused, and
  // "all SMs" (num_sms == 0) means the maximum here.
  if (prob->num_sms > SK_NOALLOC_MAX_CTAS) return SK_ERR_LIMIT;
  sk_problem q = *prob;
  if (q.num_sms <= 0) q.num_sms = SK_NOALLOC_MAX_CTAS;
  sk_resolve_auto(&q, 0, q.num_sms);
  int num_sms = 0, dev_sms = 0;
  int st = sk_resolve_grid(&q, &num_sms, &dev_sms);
  if (st != SK_OK) return st;
  SkParams p;
  memset(&p, 0, sizeof(p));
  st = sk_make_sched(&q, 0, num_sms, nullptr, &p.sched, nullptr);
  if (st != SK_OK) return st;
  if (p.sched.grid > SK_NOALLOC_MAX_CTAS) return SK_ERR_LIMIT;
  const bool nt = q.layout == SK_LAYOUT_NT;
  if (q.lda < q.K || q.ldc < q.N || q.ldb < (nt ? q.K : q.N)) return SK_ERR_SHAPE;

  // Set-up, once per device, with that device current: ask the runtime where the array
  // lives on this device.  (Also the reason the first call on a device should be made
  // outside stream capture: the lookup may load the module.)
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return sk_set_cuda_error(e);
  if (dev < 0 || dev >= 64) return SK_ERR_ARG;
  void* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    if (!g_noalloc_ptr[dev]) {
      void* ptr = nullptr;
      e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
      if (e != cudaSuccess) return sk_set_cuda_error(e);
      g_noalloc_ptr[dev] = ptr;
    }
    scratch = g_noalloc_ptr[dev];
  }
  char* base = static_cast<char*>(scratch);
  SkWorkspace w;
  w.status = reinterpret_cast<uint32_t*>(base);
  w.counters = reinterpret_cast<uint32_t*>(base + SK_WS_HEADER);
  w.done = w.counters + SK_NOALLOC_MAX_CTAS;
  w.flag_head = w.done + SK_NOALLOC_MAX_CTAS;
  w.flag_tail = w.flag_head + SK_NOALLOC_MAX_CTAS;
  w.acc_slots = reinterpret_cast<float*>(base + SK_NOALLOC_HEADER);
  w.part_slots = w.acc_slots + static_cast<size_t>(SK_NOALLOC_MAX_CTAS) * SK_SLOT_FLOATS;

  // The array keeps whatever the previous call left.  Status word, counters, flags and the
  // accumulation slots must start at zero (an earlier call that timed out may have left
  // them dirty); the partial slots need no clearing.  Stream-ordered, allocates nothing.
  cudaStream_t cs = static_cast<cudaStream_t>(stream);
  e = cudaMemsetAsync(base, 0,
                      SK_NOALLOC_HEADER + static_cast<size_t>(SK_NOALLOC_MAX_CTAS) * SK_SLOT_BYTES, cs);
  if (e != cudaSuccess) return sk_set_cuda_error(e);

  p.M = q.M; p.N = q.N; p.K = q.K;
  p.lda = q.lda; p.ldb = q.ldb; p.ldc = q.ldc;
  p.fixup = q.fixup;
  p.drop_flag_cta = q.test_drop_flag_cta - 1;
  p.timeout_ns = (q.fixup_timeout_us > 0 ? static_cast<unsigned long long>(q.fixup_timeout_us)
                                         : 2000000ULL) * 1000ULL;
  p.ws = w;
  if (nt)
    sk_gemm_f32_kernel<true><<<p.sched.grid, THREADS, 0, cs>>>(A, B, C, p);
  else
    sk_gemm_f32_kernel<false><<<p.sched.grid, THREADS, 0, cs>>>(A, B, C, p);
  e = cudaGetLastError();
  if (e != cudaSuccess) return sk_set_cuda_error(e);
  if (host_status) {
    e = cudaMemcpyAsync(host_status, w.status, sizeof(sk_status), cudaMemcpyDeviceToHost, cs);
    if (e != cudaSuccess) return sk_set_cuda_error(e);
  }
  return SK_OK;
}
