// Internal definitions shared by the kernels: workspace layout, kernel
// parameter block, device status reporting and bounded waits.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include "../../include/streamk_b200.h"
#include "sk_ptx.cuh"
#include "sk_sched.h"

// ---- workspace layout (fixed for a given SM count P) -------------------------
//   [0, 256)                 status word (sk_status) + padding
//   counters   [P] u32       atomic fixup: arrivals per split tile        (kept zero)
//   done       [P] u32       block-reduce: contributors finished reducing (kept zero)
//   flag_head  [P] u32       block-reduce: CTA's head partial is published (kept zero)
//   flag_tail  [P] u32       block-reduce: CTA's tail partial is published (kept zero)
//   acc_slots  [P]   x SLOT  fp32 accumulation slots of the atomic fixup  (kept zero)
//   part_slots [2P]  x SLOT  fp32 partials of the block-reduce fixup      (any content)
// A split tile is identified by its first contributor (the CTA that computes the
// tile's K iteration 0): a CTA starts at most one tile it does not finish (its last
// segment, the "tail") and finishes at most one tile it did not start (its first
// segment, the "head").  part_slots[2p] is CTA p's head partial, [2p+1] its tail.
constexpr size_t SK_WS_HEADER = 256;
constexpr size_t SK_SLOT_BYTES = 128 * 256 * sizeof(float);  // largest tile, fp32
constexpr size_t SK_SLOT_FLOATS = SK_SLOT_BYTES / sizeof(float);

struct SkWorkspace {
  uint32_t* status;     // 4 words
  uint32_t* counters;   // P
  uint32_t* done;       // P
  uint32_t* flag_head;  // P
  uint32_t* flag_tail;  // P
  float* acc_slots;     // P * SLOT (zero between launches)
  float* part_slots;    // 2P * SLOT
};

inline size_t sk_ws_acc_offset(int P) {
  size_t off = SK_WS_HEADER + 4 * sizeof(uint32_t) * static_cast<size_t>(P);
  return (off + 1023) & ~static_cast<size_t>(1023);
}
inline size_t sk_ws_total_bytes(int P) {
  return sk_ws_acc_offset(P) + 3 * static_cast<size_t>(P) * SK_SLOT_BYTES;
}
inline SkWorkspace sk_ws_carve(void* ws, int P) {
  char* b = static_cast<char*>(ws);
  SkWorkspace w;
  w.status = reinterpret_cast<uint32_t*>(b);
  w.counters = reinterpret_cast<uint32_t*>(b + SK_WS_HEADER);
  w.done = w.counters + P;
  w.flag_head = w.done + P;
  w.flag_tail = w.flag_head + P;
  w.acc_slots = reinterpret_cast<float*>(b + sk_ws_acc_offset(P));
  w.part_slots = reinterpret_cast<float*>(b + sk_ws_acc_offset(P) + static_cast<size_t>(P) * SK_SLOT_BYTES);
  return w;
}

// How an operand's stage tile gets into shared memory.
enum { SK_LOAD_TMA_K = 0,    // tensor map over a K-major matrix, one box per stage
       SK_LOAD_TMA_MN = 1,   // tensor map over an MN-major matrix, one 64-wide box per chunk
       SK_LOAD_IMAGE = 2,    // pre-laid-out 16 KB blocks, 1-D bulk copies
       SK_LOAD_NONE = 3 };   // produced on chip (dequantised weights)

// ---- kernel parameter block ------------------------------------------------
// The tensor-core kernels work in "kernel space": `rows` runs along the operand that
// feeds the UMMA M dimension (128 per tile), `cols` along the operand that feeds the
// UMMA N dimension (bn per tile).  Normally rows = M, cols = N.  With the operands
// swapped (short M) rows = N, cols = M and the result is stored transposed.
struct SkParams {
  int M, N, K;             // logical problem (fp32 kernel uses these)
  int lda, ldb, ldc;
  int rows, cols;          // kernel-space extents
  int transposed;          // 1: element (row, col) of the tile goes to C[col][row]
  int unit_ctas;           // CTAs that share one scheduling unit: 1, or 2 (CTA pair, 256-row tiles)
  int bn;                  // UMMA N = tile extent along cols (multiple of 16, <= 256)
  int acc_stride;          // TMEM columns between the two accumulators
  int bm;                  // rows of the UMMA M side a tile covers (tile pitch): 128, or fewer when the
                           //    weight tile is fitted to the SM count (rows beyond it hold stale data)
  int prefetch_steps;      // K steps whose boxes the producers ask L2 for before the pipeline is up
  int c_tma;               // 1: whole tiles leave through shared memory and TMA stores (tensor map of C given)
  int wide_units;          // CTA-pair kernel: 256 x 512 units walked whole after the schedule's tiles
  int wide_lag;            //    K steps the second half of a unit stays behind the first
  int kpair;               // 1: a stage is the K steps of one scale group (W4A16): two, or one at an odd
                           //    start / the end of a segment; 0: kgroup K steps per stage
  int acc_b_off;           // > 0: two MMA-issuing threads take alternate stages of a segment, the second
                           //      accumulating at this column offset; the epilogue adds the two
  int tmem_cols;           // TMEM columns allocated (power of two >= 32)
  int stages;              // shared-memory pipeline depth
  int kgroup;              // K steps (of 64) that travel together through one pipeline stage
  int w_stages;            // W4A16: depth of the dequantised-weight ring
  int q_gshift, q_groups;  // W4A16: group block of a 32-wide half step = index >> q_gshift; blocks per row
  int col_stage_bytes;     // bn * 128
  int row_tx_bytes, col_tx_bytes;   // bytes the loads of one stage deliver per operand
  int row_loader, col_loader;       // SK_LOAD_*
  uint32_t idesc;          // UMMA instruction descriptor
  int cl_per;              // SK_SCHED_CLUSTER: float4 column groups of the tile that each CTA reduces
  SkDiv cl_per_div;        // / cl_per
  SkSched sched;
  int fixup;               // SK_FIXUP_*
  int c_vec_ok;            // C rows can take 16-byte stores
  int out_bf16;            // 1: operands and result are bfloat16 (SK_FLAG_BF16), else fp16
  int drop_flag_cta;       // test hook (sk_problem.test_drop_flag_cta - 1): this CTA never publishes
                           //    its block-reduce flag; negative = off
  unsigned long long timeout_ns;
  SkWorkspace ws;
  const void* row_img;     // SK_LOAD_IMAGE sources
  const void* col_img;
  unsigned long long* trace;  // debugging: 16 timestamps per CTA, or null
};

// Fused all-gather (sk_gemm_f16_gather): every finished piece of C is also written, at the same
// row and column, into the result matrices of up to SK_MAX_PEERS other GPUs (peer-mapped
// memory; plain stores and non-multicast TMA stores).  c[i] addresses the same element of peer
// i's matrix as the kernel's C argument does of the local one; tm[i] is the tensor map over it.
//
// The same block serves the fused reduce-scatter (sk_gemm_f16_scatter): there n is the number of
// column blocks of block_cols columns each, c[j] / tm[j] the fp32 receive slot of block j's owner
// (row-major [M, block_cols], pitch block_cols), and every tile goes to exactly one of them.
constexpr int SK_MAX_TARGETS = 8;
struct alignas(64) SkPeers {
  CUtensorMap tm[SK_MAX_TARGETS];
  void* c[SK_MAX_TARGETS];
  int n;
  int block_cols;
};

// ---------------------------------------------------------------------------------------
// Small-M path (SK_SCHED_GEMV, sk_gemv.cu): how the grid is cut.  kernel_kind 1: fp16 / bf16;
// 2: W4A16 with scale groups of 128 and more (M <= 16); 3: W4A16 with groups of 32 or 64 (M <= 4).
//   fp16 / bf16: a row group is 128 weight rows; K is split across CTAs so that about four CTAs
//     per SM are in flight, in units of 256 (one warp-wide 16-byte load per row), at most 2048
//     per CTA (its activations sit in shared memory as fp32).
//   W4A16: a CTA takes 32 weight rows over all of K and cuts K into `slices` of whole steps
//     (128 of K), one per warp, whose sums meet in shared memory: 16 warps when there is at
//     most one CTA per SM, else 8, or 4 for kind 2 with more than one row of activations
//     (measured, kind 2, 4 / 8 / 16 warps: 1 x 11008 x 4096 11.3 / 11.3 / 13.9 us, 1 x 32000 x 4096
//     24.9 / 21.2 / 30.8, 8 x 11008 x 4096 12.3 / 15.0 / 15.0, 4 x 14336 x 4096 13.6 / 15.5 / 18.2;
//     kind 3, 1 x 11008 x 4096: 13.1 / 10.4 / 11.6).  Only a matrix with too
//     few rows for half of the SMs is also split across CTAs (`splits`), in pieces of at
//     least 512 of K.  (More rows per CTA with fewer slices each, 64 to 256 rows, were
//     measured with kind 3: 10-40 % slower.)
// ---------------------------------------------------------------------------------------
constexpr int SK_GEMV_MAX_M = 4;      // what the kernels take ...
constexpr int SK_GEMV_Q4_MAX_M = 16;  // ... W4A16 with scale groups of 128 and more
constexpr int SK_GEMV_AUTO_M = 1;     // what SK_SCHED_AUTO sends there: fp16 and W4A16 with small groups ...
constexpr int SK_GEMV_ROWS = 128;
constexpr int SK_GEMV_Q4_WARPS = 16;  // per CTA, at most
constexpr int SK_GEMV_Q4_SMEM_MAX = 160 * 1024;
struct SkGemvPlan {
  int groups, splits, k_per_split, grid;
  int rows, slices, k_per_slice, threads;   // W4A16; fp16: 128, 1, k_per_split, 256
};
inline bool sk_gemv_plan(int kernel_kind, int M, int N, int K, int num_sms, SkGemvPlan* out) {
  if (kernel_kind < 1 || kernel_kind > 3) return false;
  if (M < 1 || M > (kernel_kind == 2 ? SK_GEMV_Q4_MAX_M : SK_GEMV_MAX_M) || N < 1 || K < 1 || num_sms < 1) return false;
  if (kernel_kind != 1) {
    const long long groups = (static_cast<long long>(N) + 31) / 32;
    if (groups > 0x7fffffffLL / 64) return false;
    const int kblocks = (K + 63) / 64;
    const int slices0 = groups <= num_sms ? SK_GEMV_Q4_WARPS : (kernel_kind == 2 && M > 1 ? 4 : 8);
    int splits = 1;
    if (2 * groups <= num_sms) {
      splits = static_cast<int>(num_sms / groups);
      const int cap = kblocks / 8 > 1 ? kblocks / 8 : 1;
      if (splits > cap) splits = cap;
    }
    int kb_split, kb_slice, slices;
    for (;;) {   // (K blocks in pairs: a step of the kernels is 128 of K)
      kb_split = ((kblocks + splits - 1) / splits + 1) & ~1;
      kb_slice = ((kb_split + slices0 - 1) / slices0 + 1) & ~1;
      slices = (kb_split + kb_slice - 1) / kb_slice;
      // (kind 3 stages its activations: [slice][M][K of a slice] fp16)
      const long long smem = kernel_kind == 3 ? static_cast<long long>(slices) * M * kb_slice * 64 * 2 : 0;
      if (smem <= SK_GEMV_Q4_SMEM_MAX) break;
      if (splits >= kblocks) return false;
      splits *= 2;
      if (splits > kblocks) splits = kblocks;
    }
    splits = (kblocks + kb_split - 1) / kb_split;
    if (splits > 1 && groups > 4LL * num_sms) return false;   // one counter per group (the workspace has 4 per SM)
    if (groups * splits > 0x7fffffffLL) return false;
    out->groups = static_cast<int>(groups);
    out->splits = splits;
    out->k_per_split = kb_split * 64;
    out->grid = static_cast<int>(groups) * splits;
    out->rows = 32;
    out->slices = slices;
    out->k_per_slice = kb_slice * 64;
    out->threads = 32 * slices;
    return true;
  }
  const int gran = 256;
  const long long groups = (static_cast<long long>(N) + SK_GEMV_ROWS - 1) / SK_GEMV_ROWS;
  if (groups > 4LL * num_sms) return false;       // one counter per group (the workspace has 4 per SM)
  const int kunits = (K + gran - 1) / gran;
  const long long per_sm = 4;     // CTAs in flight per SM (more were measured: no gain)
  long long want = (per_sm * num_sms + groups - 1) / groups;
  if (want < 1) want = 1;
  if (want > kunits) want = kunits;
  int per = (kunits + static_cast<int>(want) - 1) / static_cast<int>(want);   // K units per split
  if (per * gran > 2048) per = 2048 / gran;
  const int splits = (kunits + per - 1) / per;
  out->groups = static_cast<int>(groups);
  out->splits = splits;
  out->k_per_split = per * gran;
  out->grid = static_cast<int>(groups) * splits;
  out->rows = SK_GEMV_ROWS;
  out->slices = 1;
  out->k_per_slice = per * gran;
  out->threads = 256;
  return true;
}
// The plan kind of an entry point's kernel kind (1: fp16, 2: W4A16) and problem flags.
inline int sk_gemv_kind(int kernel_kind, int flags) {
  if (kernel_kind != 2) return 1;
  const int grp = flags & SK_FLAG_Q4_GROUP_MASK;
  return (grp == SK_FLAG_Q4_GROUP_32 || grp == SK_FLAG_Q4_GROUP_64) ? 3 : 2;
}
struct SkWorkspace;
int sk_launch_gemv_f16(const sk_problem* prob, const void* A, const void* B, void* C, const SkWorkspace& ws,
                       int num_sms, int dev_sms, void* stream);
int sk_launch_gemv_q4(const sk_problem* prob, const void* A, const void* qblocks, const void* szblocks, void* C,
                      int gshift, int q_groups, const SkWorkspace& ws, int num_sms, int dev_sms, void* stream);

// Debugging aid, compiled in only with -DSK_TRACE (the shipped library carries none of it):
// record %globaltimer at a numbered point of this CTA's life.
__device__ __forceinline__ void sk_trace(const SkParams& p, int slot) {
#ifdef SK_TRACE
  if (p.trace) p.trace[blockIdx.x * 16 + slot] = skptx::globaltimer_ns();
#else
  (void)p; (void)slot;
#endif
}

// The same with the SM's cycle counter (finer than %globaltimer's quarter microsecond), for
// intervals inside one CTA.
__device__ __forceinline__ void sk_trace_clk(const SkParams& p, int slot) {
#ifdef SK_TRACE
  if (p.trace) p.trace[blockIdx.x * 16 + slot] = static_cast<unsigned long long>(clock64());
#else
  (void)p; (void)slot;
#endif
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
struct SkPlan {
  int swap;          // operands swapped (weights feed the UMMA M dimension)
  int bn;            // tile extent along kernel-space cols
  int rows, cols;    // kernel-space extents
  int bm;            // tile extent along kernel-space rows (128 unless fitted, see SkParams::bm)
};
int sk_set_cuda_error(cudaError_t e);
int sk_set_driver_error(int cu_result);   // a CUresult of the driver API; reported negated
int sk_resolve_grid(const sk_problem* p, int* num_sms_out, int* device_sms_out);
// kernel_kind 0: fp32 SIMT (64x64x16 tiles); 1: fp16 UMMA; 2: W4A16 UMMA.
int sk_make_sched(const sk_problem* p, int kernel_kind, int num_sms, sk_schedule_info* info,
                  SkSched* s, SkPlan* plan);
unsigned long long* sk_trace_buffer();
void sk_resolve_auto(sk_problem* q, int kernel_kind, int num_sms);
// What the fp16 entry point runs for a problem: SK_SCHED_AUTO resolved, the fused gather's
// link-bound rule applied (n_peers > 0), and the kernel chosen: *kernel_kind = 1 (single-CTA
// tiles, *units = num_sms) or 3 (CTA pairs, *units = num_sms / 2).  The one decision shared by
// sk_gemm_f16 / sk_gemm_f16_gather and the inspection call sk_schedule(kind 1).
void sk_f16_dispatch(const sk_problem* in, int num_sms, int n_peers, sk_problem* out, int* kernel_kind,
                     int* units);

// Per-device one-time set-up (kernel attributes): `fn` runs once per device ordinal per process,
// under a lock, and again only if it failed.  A device reset (cudaDeviceReset) does not clear
// the record: a process that resets a device must not use this library on it afterwards.
#include <mutex>
struct SkPerDeviceOnce {
  std::mutex m;
  bool done[64] = {false};
  template <typename F>
  cudaError_t run(F fn) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lock(m);
    if (done[dev]) return cudaSuccess;
    e = fn();
    if (e == cudaSuccess) done[dev] = true;
    return e;
  }
};

// One launch path for the tensor-core kernels: optional cluster dimension (SK_SCHED_CLUSTER, CTA
// pairs) and optional programmatic stream serialisation (SK_FLAG_PDL).
template <typename... KArgs, typename... Args>
inline cudaError_t sk_launch(void (*kernel)(KArgs...), int grid, int block, size_t smem,
                             cudaStream_t stream, int cluster, bool pdl, Args... args) {
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(block);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attrs[2];
  int n = 0;
  if (cluster > 1) {
    attrs[n].id = cudaLaunchAttributeClusterDimension;
    attrs[n].val.clusterDim.x = cluster;
    attrs[n].val.clusterDim.y = 1;
    attrs[n].val.clusterDim.z = 1;
    ++n;
  }
  if (pdl) {
    attrs[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  cfg.attrs = attrs;
  cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kernel, args...);
}
