// Internal definitions shared by the kernels: workspace layout, kernel
// parameter block, device status reporting and bounded waits.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/streamk_b200.h"
#include "sk_ptx.cuh"
#include "sk_sched.h"

// ---- workspace layout (fixed for a given SM count) -------------------------
//   [0, 256)                      status word (sk_status) + padding
//   [256, +4*P)                   counters   (atomic fixup; kept zero)
//   [.., +4*P)                    flags      (block-reduce fixup; kept zero)
//   [align 1024, +P*SLOT)         fp32 accumulation slots (atomic; kept zero)
//   [.., +P*SLOT)                 fp32 partial slots (block-reduce; any content)
// One slot belongs to one CTA: a CTA owns at most one split tile (the last
// segment of its interval) and writes at most one head partial (the first).
constexpr size_t SK_WS_HEADER = 256;
constexpr size_t SK_SLOT_BYTES = 128 * 256 * sizeof(float);  // largest tile, fp32

struct SkWorkspace {
  uint32_t* status;    // 4 words
  uint32_t* counters;  // P
  uint32_t* flags;     // P
  float* acc_slots;    // P * SLOT (zero between launches)
  float* part_slots;   // P * SLOT
};

inline size_t sk_ws_acc_offset(int P) {
  size_t off = SK_WS_HEADER + 2 * sizeof(uint32_t) * static_cast<size_t>(P);
  return (off + 1023) & ~static_cast<size_t>(1023);
}
inline size_t sk_ws_total_bytes(int P) {
  return sk_ws_acc_offset(P) + 2 * static_cast<size_t>(P) * SK_SLOT_BYTES;
}
inline SkWorkspace sk_ws_carve(void* ws, int P) {
  char* b = static_cast<char*>(ws);
  SkWorkspace w;
  w.status = reinterpret_cast<uint32_t*>(b);
  w.counters = reinterpret_cast<uint32_t*>(b + SK_WS_HEADER);
  w.flags = w.counters + P;
  w.acc_slots = reinterpret_cast<float*>(b + sk_ws_acc_offset(P));
  w.part_slots = reinterpret_cast<float*>(b + sk_ws_acc_offset(P) + static_cast<size_t>(P) * SK_SLOT_BYTES);
  return w;
}

// ---- kernel parameter block ------------------------------------------------
struct SkParams {
  int M, N, K;
  int lda, ldb, ldc;
  SkSched sched;
  int fixup;               // SK_FIXUP_*
  int c_vec_ok;            // C rows can take 16-byte stores
  int a_tx_bytes;          // bytes one TMA load of the A stage tile delivers
  int drop_flag_cta;       // test hook, -1 = off
  unsigned long long timeout_ns;
  SkWorkspace ws;
  unsigned long long* trace;  // debugging: 8 timestamps per CTA, or null
};

// Debugging aid: record %globaltimer at a numbered point of this CTA's life.
__device__ __forceinline__ void sk_trace(const SkParams& p, int slot) {
  if (p.trace) p.trace[blockIdx.x * 8 + slot] = skptx::globaltimer_ns();
}

// First reporter wins; later errors keep the first record.
__device__ __forceinline__ void sk_report(uint32_t* status, uint32_t code, uint32_t d0, uint32_t d1) {
  if (atomicCAS(status, 0u, code) == 0u) {
    status[1] = blockIdx.x;
    status[2] = d0;
    status[3] = d1;
    __threadfence();
  }
}

// Bounded spin on a global flag written by another CTA.  Returns false when the
// time limit ran out (the caller reports and carries on without the data).
__device__ __forceinline__ bool sk_wait_flag(const uint32_t* flag, unsigned long long timeout_ns) {
  if (skptx::ld_acquire_u32(flag) != 0u) return true;
  const unsigned long long t0 = skptx::globaltimer_ns();
  unsigned spins = 0;
  for (;;) {
    if (skptx::ld_acquire_u32(flag) != 0u) return true;
    __nanosleep(spins < 16 ? 32 : 256);
    if ((++spins & 15u) == 0u && skptx::globaltimer_ns() - t0 > timeout_ns) return false;
  }
}

// Host-side helpers implemented in sk_api.cu.
int sk_set_cuda_error(cudaError_t e);
int sk_resolve_grid(const sk_problem* p, int* num_sms_out, int* device_sms_out);
int sk_make_sched(const sk_problem* p, int kernel_kind, int num_sms, sk_schedule_info* info, SkSched* s);
unsigned long long* sk_trace_buffer();
