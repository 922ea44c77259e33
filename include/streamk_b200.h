/*
 * streamk_b200 — C ABI of the B200 (sm_100a) Stream-K GEMM library.
 *
 * Every function is extern "C", takes plain pointers and sizes, returns an int
 * status (0 = SK_OK), never throws, never synchronises the device and — except
 * where a comment says otherwise — never allocates.  All device pointers must
 * belong to the device that is current on the calling thread.  `stream` is a
 * cudaStream_t passed as void* (NULL = the legacy default stream).
 *
 * The reference (LeiWang1999/Stream-k.tvm) has no FFI: each script builds a TVM
 * prim_func and calls `tl_mod(A, B, C)` with caller-owned, pre-zeroed CUDA
 * tensors.  Each entry point below names the reference call it stands in for.
 */
#ifndef STREAMK_B200_H_
#define STREAMK_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ------------------------------------------------------ */
enum {
  SK_OK = 0,
  SK_ERR_ARCH = 1,          /* device is not compute capability 10.x           */
  SK_ERR_ALIGN = 2,         /* pointer / leading dimension alignment           */
  SK_ERR_SHAPE = 3,         /* non-positive or unsupported extent              */
  SK_ERR_WORKSPACE = 4,     /* workspace missing or too small                  */
  SK_ERR_LAUNCH = 5,        /* CUDA runtime / driver error (see sk_last_cuda_error) */
  SK_ERR_FIXUP_TIMEOUT = 6, /* device: a tile owner gave up waiting on a peer  */
  SK_ERR_PIPE_TIMEOUT = 7,  /* device: an mbarrier wait ran out                */
  SK_ERR_ARG = 8,           /* bad enum value / null pointer                   */
  SK_ERR_LIMIT = 9          /* size beyond a stated maximum                    */
};

/* ---- enums ------------------------------------------------------------- */
enum { SK_LAYOUT_NN = 0,      /* B is [K,N] row-major  (streamk_fp32.py:74, streamk_fp16_nn.py)   */
       SK_LAYOUT_NT = 1,      /* B is [N,K] row-major  (streamk_fp16.py:128, streamk_fp16_nt.py)  */
       SK_LAYOUT_LADDER = 2   /* B pre-laid-out by sk_prepack_ladder (streamk_fp16_ladder.py:153) */ };

enum { SK_SCHED_STREAMK = 0,        /* every tile is Stream-K'd                                   */
       SK_SCHED_HYBRID = 1,         /* reference order: SK tiles first, then DP waves
                                       (streamk_fp16.py:98-113, 353-371)                          */
       SK_SCHED_HYBRID_DP_FIRST = 2,/* same tile split, DP waves first, SK remainder last         */
       SK_SCHED_DP = 3,             /* plain data-parallel: one whole tile per CTA per wave       */
       SK_SCHED_AUTO = 4,           /* the library picks schedule (and open tile sizes) by shape  */
       SK_SCHED_CLUSTER = 5,        /* split-K inside a thread-block cluster: every tile is walked
                                       by the 2, 4 or 8 CTAs of one cluster (the largest size with
                                       tiles x size <= num_sms), CTA r taking K iterations
                                       [r*I/size, (r+1)*I/size); the partial tiles meet in the
                                       cluster's distributed shared memory and are summed in CTA
                                       order, so no workspace traffic and a bitwise reproducible
                                       result.  fp16 and W4A16 entry points; `fixup` is ignored.  No
                                       counterpart in the reference.                              */
       SK_SCHED_GEMV = 6            /* A few rows of activations only: the product as one stream of
                                       the weights through small CTAs, without tensor memory,
                                       clusters or workspace fix-ups.  fp16 / bf16 NT and W4A16 with
                                       scale groups of 32 or 64: M <= 4, on the CUDA cores.  W4A16
                                       with groups of 128 and more: M <= 16, register-level
                                       tensor-core instructions on the packed nibbles.  Partial sums
                                       meet in a fixed order (bitwise reproducible); `fixup`,
                                       tile_m, tile_n, group_m and num_sms < device are ignored;
                                       fp16: N <= 512 x the SM count.  What SK_SCHED_AUTO picks for
                                       fp16 at M = 1 and for W4A16 up to M = 8 (groups of 128 and
                                       more; up to 16 when N <= 32 x the SM count; M = 1 with
                                       smaller groups).  No counterpart in the
                                       reference, whose kernels are tensor-core tiled at every M. */ };

enum { SK_FIXUP_ATOMIC = 0,        /* fp32 red.global.add into a self-cleaning workspace
                                      (replaces T.atomic_addx2, streamk_fp16.py:248-255)          */
       SK_FIXUP_BLOCK_REDUCE = 1   /* flag-synchronised, fixed-order, bitwise reproducible        */ };

/* ---- problem description ------------------------------------------------ */
typedef struct sk_problem {
  int32_t M, N, K;
  int32_t lda, ldb, ldc;      /* leading dimensions in elements (row-major)   */
  int32_t layout;             /* SK_LAYOUT_*                                  */
  int32_t schedule;           /* SK_SCHED_*                                   */
  int32_t fixup;              /* SK_FIXUP_*                                   */
  int32_t tile_m;             /* 0 = choose; 128 = M feeds the UMMA M dimension;
                                 16..256 (multiple of 16) = operands swapped: the
                                 weights feed the UMMA M dimension and the tile
                                 spans tile_m rows of C (for short M).  fp16 NT,
                                 256: the CTA-pair kernel (256-row tiles, tile_n a
                                 multiple of 16 from 32, default 256)           */
  int32_t tile_n;             /* 0 = choose; columns of C per tile: a multiple of 16 up
                                 to 256 (W4A16: 128).  Operands swapped: weight rows
                                 per tile, 128, or for fp16 NT a multiple of 8 from
                                 16 to 128                                      */
  int32_t num_sms;            /* 0 = all SMs of the device; else grid size    */
  int32_t group_m;            /* 0 = choose; tile rasterisation group height  */
  int32_t fixup_timeout_us;   /* 0 = default (2 s); bound of every device wait */
  int32_t test_drop_flag_cta; /* 0 (or negative) = off, so a zero-initialised struct is
                                 an ordinary problem.  Test only: n > 0 makes CTA n - 1
                                 never publish its block-reduce flag, so its tile owner
                                 runs into the bounded wait and reports a timeout. */
  int32_t flags;              /* SK_FLAG_* bits                                */
} sk_problem;

/* sk_problem.flags */
enum { SK_FLAG_PDL = 1, /* fp16 / W4A16 entry points: launch with programmatic stream
                          serialisation.  The kernel's start-up (mbarrier set-up, tensor-memory
                          allocation, scheduling arithmetic) may then overlap the tail of the
                          kernel before it in the stream if that kernel lets its dependents go
                          early (these kernels do, at entry); nothing touches global memory
                          before the preceding kernel has completed (griddepcontrol.wait), so
                          results and stream order are unchanged.  Worth 1-2 us per launch in a
                          chain of small GEMMs.                                            */
       SK_FLAG_BF16 = 4, /* sk_gemm_f16 / sk_gemm_f16_gather / sk_prepack_ladder images: A, B and C hold
                          bfloat16 instead of fp16 (same layouts, same kernels: the UMMA reads the
                          operands as bf16, accumulates in fp32, and the epilogue rounds to bf16).
                          No counterpart in the reference (fp16 only); its README's dtype TODO.  */
       /* sk_gemm_w4a16: group size of the packed image's scales / zero-points along K (two-bit
          field; the default, 0, is 128).  Must match what sk_prepack_q4_ex was given.         */
       SK_FLAG_Q4_GROUP_32 = 0x100, SK_FLAG_Q4_GROUP_64 = 0x200, SK_FLAG_Q4_PER_CHANNEL = 0x300,
       SK_FLAG_Q4_GROUP_MASK = 0x300,
       SK_FLAG_NO_TABLE = 2 /* SK_SCHED_AUTO: resolve by the built-in rules only, without
                          consulting the table of tuned shapes (what the offline tuner itself
                          uses to time the rules' choice).                                 */ };

/* Host scheduler result: the integers of streamk_fp16.py:83-113 plus the
 * derived per-CTA split, exposed so callers and tests can inspect them.     */
typedef struct sk_schedule_info {
  int32_t tile_m, tile_n, tile_k;
  int32_t tiles_m, tiles_n, total_tiles, iters_per_tile;
  int32_t sk_tiles, dp_tiles;
  int32_t grid;                /* persistent CTAs launched                    */
  int32_t sk_iters_per_cta;    /* "streamk_full_tiles"  (floor)               */
  int32_t sk_iters_rem;        /* "streamk_partial_tiles" (CTAs with one more)*/
  int32_t dp_waves;            /* ceil(dp_tiles / grid)                       */
  int32_t dp_first;
  int32_t group_m;
  int32_t swap_ab;             /* 1: weights feed the UMMA M dimension          */
  int32_t schedule;            /* the schedule used (SK_SCHED_AUTO resolved)    */
  int32_t cluster;             /* SK_SCHED_CLUSTER: CTAs per tile; else 0       */
  int32_t wide_units;          /* CTA-pair kernel, hybrid schedule: the dp_tiles are walked as
                                  this many units of two column-adjacent tiles (the first
                                  wide_units units of the rasterised tiles_m x tiles_n/2 grid);
                                  Stream-K tile t is then half t & 1 of unit wide_units + t/2  */
} sk_schedule_info;

typedef struct sk_device_info {
  int32_t cc_major, cc_minor;
  int32_t num_sms;
  int32_t max_smem_optin;
  int64_t l2_bytes;
  int64_t total_mem;
} sk_device_info;

typedef struct sk_status {
  uint32_t code;     /* SK_OK, SK_ERR_FIXUP_TIMEOUT or SK_ERR_PIPE_TIMEOUT     */
  uint32_t cta;      /* CTA that reported                                      */
  uint32_t detail0;  /* fixup: tile id      pipe: barrier id                   */
  uint32_t detail1;  /* fixup: awaited CTA  pipe: role                         */
} sk_status;

/* ---- library / device --------------------------------------------------- */
const char* sk_version(void);
const char* sk_status_string(int status);
/* Cause of the most recent SK_ERR_LAUNCH on this thread: > 0 a cudaError_t of the runtime,
 * < 0 the negated CUresult of a driver call (tensor-map encoding). */
int sk_last_cuda_error(void);
int sk_query(int device, sk_device_info* out);

/* Debugging aid, no counterpart in the reference.  Works only in a library compiled with
 * -DSK_TRACE (the build recipe's STREAMK_B200_TRACE=1); the ordinary build carries no tracing
 * code in its kernels and this call then accepts NULL only (SK_ERR_ARG otherwise).  While
 * `buf` (device memory, 128 bytes per SM) is set, tensor-core launches record %globaltimer
 * stamps per CTA (16 slots of 8 bytes): 0 entry, 1 set-up done, 2 first TMA issued, 3 first
 * stage consumed, 4 last MMA issued, 5 first accumulator ready, 6 epilogue done, 7 exit,
 * 8 fixup flags seen, 9 / 10 first / second split tile reduced, 11 flags re-armed.  One
 * pointer per process: set it while no launch is in flight.  NULL switches it off.       */
int sk_debug_set_trace(void* buf);

/* ---- scheduler (host only, no GPU needed) ------------------------------- */
/* kernel_kind: 0 = fp32 SIMT tiles (64x64x16), 1 = what sk_gemm_f16 runs for the problem
 * (single-CTA UMMA tiles, or the CTA-pair kernel over num_sms / 2 pairs: the info then
 * describes 256-row tiles), 2 = W4A16 UMMA tiles (tile_m x tile_n x 64), 3 = the CTA-pair
 * kernel with num_sms pairs.  Mirrors streamk_fp16.py:83-113 for SK_SCHED_HYBRID. */
int sk_schedule(const sk_problem* p, int kernel_kind, int num_sms, sk_schedule_info* out);
/* The same question for sk_gemm_f16_gather with n_peers peers (a link-bound gather makes the
 * library drop the 256 x 512 units and, if the schedule was left to it, run data-parallel). */
int sk_schedule_gather(const sk_problem* p, int n_peers, int num_sms, sk_schedule_info* out);
/* Iteration interval [begin,end) of CTA `cta` (streamk_fp16.py:176-181). */
int sk_cta_interval(const sk_schedule_info* s, int cta, int64_t* begin, int64_t* end);
/* Tile id -> (tile row, tile column) under the grouped rasterisation. */
int sk_tile_coords(const sk_schedule_info* s, int tile, int* tile_m, int* tile_n);

/* ---- workspace ----------------------------------------------------------- */
/* One workspace serves every kernel of this library on one device; it holds
 * the status word, per-CTA counters and flags, the zero-kept fp32 accumulation
 * slots of the atomic fixup and the partial slots of the block-reduce fixup.
 * Size depends only on the SM count.  The caller allocates it (cudaMalloc or a
 * torch tensor), calls sk_workspace_init once, and must not share it between
 * launches that can overlap on the GPU.  Kernels leave it clean; after a
 * reported device error call sk_workspace_init again.                        */
size_t sk_workspace_bytes(int num_sms);
int sk_workspace_init(void* ws, size_t bytes, void* stream);
/* Asynchronously copies the 16-byte status word into host_out (pinned memory
 * recommended); valid after the stream is synchronised.                      */
int sk_poll_status(const void* ws, sk_status* host_out, void* stream);

/* ---- GEMM entry points --------------------------------------------------- */
/* C[M,N] = A[M,K] . B, fp32 in / fp32 accumulate / fp32 out, CUDA-core FFMA
 * (no TF32).  Replaces tl_mod(A, B, C) of streamk_fp32.py:57-202 (layout NN)
 * and accepts NT as well.  C need not be zeroed.                             */
int sk_gemm_f32(const sk_problem* p, const float* A, const float* B, float* C,
                void* ws, size_t ws_bytes, void* stream);

/* No counterpart in the reference.  sk_gemm_f32 for callers that cannot hand over a
 * workspace because they must not allocate: hosts with a memory budget fixed at start-up,
 * code in regions where cudaMalloc is forbidden, plugin interfaces that pass operands
 * only.  The fixup scratch is a fixed array inside the library image (about 6 MB, held by
 * every GPU that loads the library until the process exits), sized for 16 persistent
 * CTAs: num_sms == 0 means 16 here and num_sms > 16 is refused with SK_ERR_LIMIT.  The
 * call allocates nothing (no cudaMalloc / cudaFree, no allocating library routine).  The
 * first call on a device looks the array's address up (cudaGetSymbolAddress); make that
 * first call outside stream capture.  All calls on a device share the one array: calls
 * that can overlap on the GPU (different streams, different host threads) race and must
 * be serialised by the caller.  host_status may be NULL; otherwise the device status
 * word is copied into it asynchronously (valid once the stream is synchronised): pass
 * pinned host memory -- with pageable memory the copy makes the call wait for the kernel,
 * and it cannot be recorded into a stream capture -- or NULL and read the status some
 * other way.  The per-device address look-up is remembered for the life of the process;
 * a process that resets a device (cudaDeviceReset) must not call this on it afterwards. */
int sk_gemm_f32_noalloc(const sk_problem* p, const float* A, const float* B, float* C,
                        sk_status* host_status, void* stream);

/* C[M,N] = A[M,K] . op(B), fp16 in / fp32 accumulate in TMEM / fp16 out on
 * tcgen05 tensor cores.  Replaces tl_mod(A, B, C) of streamk_fp16.py:116-387
 * (NT), streamk_fp16_nn.py (NN), streamk_fp16_block_reduce.py and
 * streamk_fp16_ladder*.py (LADDER: B from sk_prepack_ladder).  A, B 16-byte
 * aligned, lda/ldb multiples of 8.  C need not be zeroed.                    */
int sk_gemm_f16(const sk_problem* p, const void* A, const void* B, void* C,
                void* ws, size_t ws_bytes, void* stream);

/* sk_gemm_f16 fused with the all-gather of an N-sharded product (the reference is a
 * single-GPU study; this is the column-sharded configuration's collective).  Every GPU of
 * a group holds the full result matrix [M, N_total] and computes one column block of it.
 * C addresses element (0, first column of this GPU's block) of the local matrix and
 * peers[i] the same element of peer i's matrix (peer-mapped device memory, e.g. from
 * sk_peer_open; same ldc everywhere).  The kernel's epilogue writes every finished tile
 * to C and to all peers in the order given (plain peer stores and TMA stores without
 * multicast, no device-side wait on another GPU), so the transfer overlaps the mainloop
 * tile by tile.  The call is stream-ordered like sk_gemm_f16; the gathered matrix is
 * complete on a GPU once ALL GPUs' kernels have finished: the caller places a host or
 * NCCL barrier after the call before reading foreign blocks, and one before the next call
 * overwrites them.  Needs the CTA-pair kernel (NT layout, tile_m = 256 or a problem large
 * enough that the library picks it: SK_ERR_SHAPE otherwise), C and peers 16-byte aligned,
 * ldc a multiple of 8, n_peers <= SK_MAX_PEERS.  n_peers == 0 is sk_gemm_f16.           */
enum { SK_MAX_PEERS = 7 };
int sk_gemm_f16_gather(const sk_problem* p, const void* A, const void* B, void* C,
                       void* const* peers, int n_peers, void* ws, size_t ws_bytes, void* stream);

/* sk_gemm_f16 for a K-SHARDED product, fused with the reduce-scatter of the partial sums (the
 * other collective of a tensor-parallel linear layer; no counterpart in the single-GPU
 * reference).  GPU g of G holds A[:, K_g] and B[:, K_g] and computes the partial product
 * P_g = A_g . B_g^T over the full [M, N]; GPU j is to end up with columns [j N/G, (j+1) N/G) of
 * the sum.  The kernel's epilogue writes every tile of P_g, as fp32, straight into dst[j], the
 * receive slot that the owner j of the tile's column block keeps for this sender: row-major
 * [M, N/G] fp32, pitch N/G, 16-byte aligned, local or peer-mapped memory (sk_peer_open).  Plain
 * TMA stores without multicast, no device-side wait on another GPU: the transfer runs under the
 * mainloop tile by tile.  Once every GPU's kernel has finished (a host or NCCL barrier placed by
 * the caller), each owner adds its G slots in ascending sender order with sk_reduce_partials --
 * a fixed order, so the result is bitwise reproducible.  Runs the CTA-pair kernel with whole
 * tiles (NT layout, even SM count, N/G a multiple of the tile width: tile_n, default 256, and
 * of 4; SK_ERR_SHAPE otherwise); prob->ldc and prob->schedule are ignored, n_blocks <= 8.     */
int sk_gemm_f16_scatter(const sk_problem* p, const void* A, const void* B, void* const* dst, int n_blocks,
                        void* ws, size_t ws_bytes, void* stream);
/* C[M, Nb] (fp16, or bf16 with SK_FLAG_BF16 in flags; pitch ldc, a multiple of 4) = the sum, in
 * ascending order, of n_parts fp32 matrices [M, Nb] stored back to back at `parts`.          */
int sk_reduce_partials(const void* parts, int n_parts, int M, int Nb, void* C, int ldc, int flags,
                       void* stream);

/* Device memory other processes of this machine can map (CUDA IPC), for the matrices
 * sk_gemm_f16_gather writes into.  sk_peer_alloc: cudaMalloc + export; `handle` receives
 * SK_PEER_HANDLE_BYTES opaque bytes to send to the other processes (any channel).
 * sk_peer_open maps a handle received from another process (peer access is enabled as
 * needed) and returns a device pointer valid in this process; sk_peer_close unmaps it;
 * sk_peer_free releases an allocation of sk_peer_alloc (after every peer closed it).    */
enum { SK_PEER_HANDLE_BYTES = 64 };
int sk_peer_alloc(size_t bytes, void** ptr, void* handle);
int sk_peer_open(const void* handle, void** ptr);
int sk_peer_close(void* ptr);
int sk_peer_free(void* ptr);

/* Bytes of the pre-laid-out image of an fp16 weight B[N,K]. */
size_t sk_ladder_bytes(int N, int K);
/* One-time re-layout of B[N,K] (row-major fp16, ldb elements) into the image
 * the LADDER mainloop streams with 1-D bulk copies.  Replaces
 * bitblas.ops.LadderPermutate on CPU (streamk_fp16_ladder.py:468-477).        */
int sk_prepack_ladder(const void* B, int N, int K, int ldb, void* out, size_t out_bytes,
                      void* stream);

/* W4A16: C[M,N] = A[M,K] . W^T with W = (q - z) * s, q uint4, per-group z
 * (uint4 stored as uint8) and fp16 s, group size 128 along K.
 * Bytes of the packed image produced by sk_prepack_q4.                        */
size_t sk_q4_bytes(int N, int K);
/* qweight: int32 [N, K/8], nibble j of word w of row n is k = 8w + j (byte
 * identical to the reference's int8 [N,K/2] low-nibble-first storage,
 * streamk_fp16_ladder_block_reduce_q4.py:545-554).  scales fp16 [N, K/128] or
 * NULL (=1), zeros uint8 [N, K/128] or NULL (=0).  Replaces LadderPermutate +
 * LOP3Permutate on CPU (…q4.py:568-595).  K must be a multiple of 128.        */
int sk_prepack_q4(const void* qweight, const void* scales, const void* zeros, int N, int K,
                  void* out, size_t out_bytes, void* stream);
/* W[N,K] fp16 = dequantised image (bit-exact (q - z) * s with fp16 rounding). */
int sk_dequant_q4(const void* packed, int N, int K, void* W, int ldw, void* stream);
/* Further quantisation formats (the reference stops at plain uint4 and lists the rest as open
 * work, README.md:20-21).  group_size: 32, 64, 128, or 0 / K for one group per weight row
 * (per-channel scales); scales / zeros are then [N, K / group_size] (or [N, 1]).  is_signed: the
 * nibbles are two's-complement int4 and the format is symmetric, W = q * s (zeros must be NULL);
 * stored as q + 8 with zero-point 8, which is the same arithmetic exactly.  The GEMM is told
 * the group size through SK_FLAG_Q4_GROUP_* in sk_problem.flags.                            */
size_t sk_q4_bytes_ex(int N, int K, int group_size);
int sk_prepack_q4_ex(const void* qweight, const void* scales, const void* zeros, int N, int K,
                     int group_size, int is_signed, void* out, size_t out_bytes, void* stream);
int sk_dequant_q4_ex(const void* packed, int N, int K, int group_size, void* W, int ldw, void* stream);
/* Replaces tl_mod(A, QLB, C) of streamk_fp16_ladder_block_reduce_q4.py:143-599. */
int sk_gemm_w4a16(const sk_problem* p, const void* A, const void* packed, void* C,
                  void* ws, size_t ws_bytes, void* stream);

/* Pitched copy, stream-ordered (cudaMemcpy2DAsync, direction inferred from the pointers):
 * `rows` rows of `width_bytes` bytes, row pitches in bytes.  Used by the Python layer's
 * host-buffer entry point to move column slabs of a row-major host matrix at DMA speed.
 * No counterpart in the reference (its scripts keep everything on the device).            */
int sk_memcpy2d_async(void* dst, size_t dst_pitch, const void* src, size_t src_pitch,
                      size_t width_bytes, size_t rows, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* STREAMK_B200_H_ */
