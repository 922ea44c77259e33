// Library-level C ABI: version, device query, host scheduler, workspace.
#include <string.h>

#include <atomic>

#include "sk_common.cuh"

static thread_local int g_last_cuda_error = 0;

int sk_set_cuda_error(cudaError_t e) {
  g_last_cuda_error = static_cast<int>(e);
  return SK_ERR_LAUNCH;
}

// A CUresult of the driver API (tensor-map encoding) is kept negated, so that
// sk_last_cuda_error tells the two apart: > 0 cudaError_t, < 0 -CUresult.
int sk_set_driver_error(int cu_result) {
  g_last_cuda_error = -cu_result;
  return SK_ERR_LAUNCH;
}

// Debugging aid (not part of the reference surface), present only in a library built with
// -DSK_TRACE: later launches of the tensor-core kernels record up to sixteen %globaltimer
// stamps per CTA into `buf` (device memory, 128 bytes per SM); NULL switches it off.  One
// pointer for the process: a test-only switch, to be set while no launch is in flight.
#ifdef SK_TRACE
static std::atomic<unsigned long long*> g_trace{nullptr};
unsigned long long* sk_trace_buffer() { return g_trace.load(std::memory_order_acquire); }
extern "C" int sk_debug_set_trace(void* buf) {
  g_trace.store(static_cast<unsigned long long*>(buf), std::memory_order_release);
  return SK_OK;
}
#else
unsigned long long* sk_trace_buffer() { return nullptr; }
extern "C" int sk_debug_set_trace(void* buf) { return buf ? SK_ERR_ARG : SK_OK; }
#endif

extern "C" const char* sk_version(void) { return "streamk_b200 0.1 (sm_100a)"; }

extern "C" int sk_last_cuda_error(void) { return g_last_cuda_error; }

extern "C" const char* sk_status_string(int status) {
  switch (status) {
    case SK_OK: return "ok";
    case SK_ERR_ARCH: return "device is not an sm_100 GPU";
    case SK_ERR_ALIGN: return "pointer or leading dimension is not aligned as required";
    case SK_ERR_SHAPE: return "unsupported problem shape";
    case SK_ERR_WORKSPACE: return "workspace missing or too small";
    case SK_ERR_LAUNCH: return "CUDA error (see sk_last_cuda_error)";
    case SK_ERR_FIXUP_TIMEOUT: return "device: tile owner timed out waiting for a peer partial";
    case SK_ERR_PIPE_TIMEOUT: return "device: pipeline barrier wait timed out";
    case SK_ERR_ARG: return "invalid argument";
    case SK_ERR_LIMIT: return "size beyond the supported maximum";
    default: return "unknown status";
  }
}

extern "C" int sk_query(int device, sk_device_info* out) {
  if (!out) return SK_ERR_ARG;
  cudaDeviceProp prop;
  cudaError_t e = cudaGetDeviceProperties(&prop, device);
  if (e != cudaSuccess) return sk_set_cuda_error(e);
  out->cc_major = prop.major;
  out->cc_minor = prop.minor;
  out->num_sms = prop.multiProcessorCount;
  out->max_smem_optin = static_cast<int32_t>(prop.sharedMemPerBlockOptin);
  out->l2_bytes = prop.l2CacheSize;
  out->total_mem = static_cast<int64_t>(prop.totalGlobalMem);
  return prop.major == 10 ? SK_OK : SK_ERR_ARCH;
}

// SM count of the current device (cached per device) and the grid bound asked for.
int sk_resolve_grid(const sk_problem* p, int* num_sms_out, int* device_sms_out) {
  static std::atomic<int> cached[64];   // zero-initialised; racing first calls store the same value
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return sk_set_cuda_error(e);
  if (dev < 0 || dev >= 64) return SK_ERR_ARG;
  int sms = cached[dev].load(std::memory_order_relaxed);
  if (sms == 0) {
    int major = 0;
    e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return sk_set_cuda_error(e);
    e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    if (e != cudaSuccess) return sk_set_cuda_error(e);
    if (major != 10) return SK_ERR_ARCH;
    cached[dev].store(sms, std::memory_order_relaxed);
  }
  *device_sms_out = sms;
  if (p->num_sms > 0) {
    if (p->num_sms > sms) return SK_ERR_LIMIT;  // co-residency of all CTAs is required
    sms = p->num_sms;
  }
  *num_sms_out = sms;
  return SK_OK;
}

// Chooses the tile shape and whether the operands are swapped.
//   kernel_kind 0 (fp32 SIMT): 64 x 64 x 16 tiles, never swapped.
//   kernel_kind 3 (fp16 UMMA, CTA pairs): 256 x 256 x 64 tiles, one per pair of CTAs;
//   `num_sms` is then the number of pairs.
//   kernel_kind 1/2 (fp16 / W4A16 UMMA): the UMMA M dimension is always 128.  Normally it
//   runs along M and the tile is 128 x tile_n (128 or 256).  For short M the weights take
//   the UMMA M dimension instead (128 along N) and the tile spans tile_m = M rounded up to
//   16 along M: no tensor-core work, shared memory or epilogue lanes are spent on padding.
static int make_plan(const sk_problem* p, int kernel_kind, int num_sms, SkPlan* plan) {
  if (kernel_kind == 0) {
    plan->swap = 0; plan->bn = 64; plan->bm = 64; plan->rows = p->M; plan->cols = p->N;
    return SK_OK;
  }
  if (kernel_kind == 3) {   // CTA pairs: 256 x 256 tiles, or 256 x tile_n (a multiple of 16)
    int tn = p->tile_n ? p->tile_n : 256;
    if (tn < 32 || tn > 256 || (tn & 15) != 0) return SK_ERR_ARG;
    plan->swap = 0; plan->bn = tn; plan->bm = 128; plan->rows = p->M; plan->cols = p->N;
    return SK_OK;
  }
  int tm = p->tile_m, tn = p->tile_n;
  if (tm < 0 || tn < 0) return SK_ERR_ARG;
  if (kernel_kind == 2) {
    // W4A16: the weights always feed the UMMA M dimension (their dequantised form is the
    // tensor-memory A operand): 128 weight rows per tile, tile_m = 16 .. 128 rows of C.  Left
    // open, M is cut into equal tiles of at most 128 rows.
    if (tn != 0 && tn != 128) return SK_ERR_ARG;
    if (tm == 0) {
      // (the cluster schedule's exchange buffers leave room for tiles of at most 112 rows)
      const int cap = p->schedule == SK_SCHED_CLUSTER ? 112 : 128;
      const int parts = (p->M + cap - 1) / cap;
      tm = ((p->M + parts - 1) / parts + 15) & ~15;
    }
    if (tm < 16 || tm > 128 || (tm & 15) != 0) return SK_ERR_ARG;
    plan->swap = 1; plan->bn = tm; plan->bm = 128; plan->rows = p->N; plan->cols = p->M;
    return SK_OK;
  }
  bool swap;
  if (tm == 0 && tn == 0) swap = p->M <= 64;
  else if (tm != 0 && tm != 128) swap = true;
  else if (tm == 128 && tn == 0 && p->M <= 64) swap = false;
  else swap = false;
  if (swap) {
    // tile_n = weight rows per tile: 128, or for fp16 NT any multiple of 8 from 16 (the TMA
    // box then has fewer rows; the UMMA still spans 128, the rest of its rows is ignored)
    if (tn == 0) tn = 128;
    const bool fitted_ok = kernel_kind == 1 && p->layout == SK_LAYOUT_NT;
    if (tn != 128 && !(fitted_ok && tn >= 16 && tn < 128 && (tn & 7) == 0)) return SK_ERR_ARG;
    if (tm == 0) tm = (p->M + 15) & ~15;
    if (tm < 16 || tm > 256 || (tm & 15) != 0) return SK_ERR_ARG;
    plan->swap = 1; plan->bn = tm; plan->bm = tn; plan->rows = p->N; plan->cols = p->M;
    return SK_OK;
  }
  if (tn == 0) {
    // Wide tiles halve shared-memory traffic per flop; use them once there is
    // enough work to fill every SM twice over, else favour granularity.
    const long long t256 = static_cast<long long>((p->M + 127) / 128) * ((p->N + 255) / 256);
    tn = (t256 >= 2LL * num_sms) ? 256 : 128;
  }
  // any multiple of 16 up to 256 (NN and ladder weights come in 128-row units: checked by the caller)
  if (tn < 16 || tn > 256 || (tn & 15) != 0) return SK_ERR_ARG;
  plan->swap = 0; plan->bn = tn; plan->bm = 128; plan->rows = p->M; plan->cols = p->N;
  return SK_OK;
}

// SK_SCHED_AUTO: replace the schedule (and, if the caller left them open, the tile) by the
// choice that measured best on B200 for this kind of shape.  The rules of thumb behind it:
//  * a fixup costs a few microseconds of L2 round trips, so when whole tiles alone can keep
//    most SMs busy, run them data-parallel with the tile width fitted to the SM count;
//  * otherwise every SM has to stream (one SM's share of a weight stream stays below ~50 GB/s): Stream-K;
//  * large problems: the reference's hybrid split.
// Shapes for which the offline tuner (`python bench.py --tune FILE`, which times the candidates
// and rejects any whose result is out of tolerance) found something better than the rules
// below.  Consulted first, for exact (kind, M, N, K, SM count) matches with open tile sizes.
namespace {
struct SkTuned { int kind, M, N, K, sms, schedule, tile_m, tile_n; };
const SkTuned kTuned[] = {
#include "sk_tuned_table.inc"
    {-1, 0, 0, 0, 0, 0, 0, 0}};
}  // namespace

void sk_resolve_auto(sk_problem* q, int kernel_kind, int num_sms) {
  if (q->schedule != SK_SCHED_AUTO) return;
  q->schedule = SK_SCHED_HYBRID;
  if (kernel_kind == 0 || kernel_kind == 3) return;
  const bool tiles_open = q->tile_m == 0 && q->tile_n == 0;
  // (the tuner times the NT entry point; NN and ladder weights come in 128-row units and keep the rules)
  if (tiles_open && (q->flags & SK_FLAG_NO_TABLE) == 0 && (kernel_kind != 1 || q->layout == SK_LAYOUT_NT)) {
    for (const SkTuned* t = kTuned; t->kind >= 0; ++t) {
      if (t->kind != kernel_kind || t->M != q->M || t->N != q->N || t->K != q->K || t->sms != num_sms) continue;
      sk_problem c = *q;
      c.schedule = t->schedule; c.tile_m = t->tile_m; c.tile_n = t->tile_n;
      // (a row that no longer plans -- the kernels changed since it was written -- is ignored)
      const bool pairs = kernel_kind == 1 && t->tile_m == 256;
      if (sk_make_sched(&c, pairs ? 3 : kernel_kind, pairs ? num_sms / 2 : num_sms, nullptr, nullptr, nullptr) == SK_OK) {
        *q = c;
        return;
      }
    }
  }
  const int gemv_kind = sk_gemv_kind(kernel_kind, q->flags);
  // (W4A16: 9 to 16 rows cost the small-M kernel twice the instructions of 1 to 8: only where the
  // launch is short enough to be bound by latencies, at most one 32-row CTA per SM)
  const int gemv_m = gemv_kind != 2 ? SK_GEMV_AUTO_M : (q->N <= 32LL * num_sms ? SK_GEMV_Q4_MAX_M : 8);
  if (tiles_open && q->M <= gemv_m && (kernel_kind == 2 || q->layout == SK_LAYOUT_NT)) {
    // Few rows of activations: the weights stream once through a kernel without the tensor-core
    // kernels' fixed costs (tensor-memory allocation, mbarrier rings, a cluster exchange or a
    // workspace fix-up).  W4A16 with scale groups of 128 and more, whose small-M kernel takes
    // eight rows for the price of one (measured L2-cold at 4096 x 4096, 11008 x 4096,
    // 4096 x 11008: M = 1 5.9 / 11.2 / 11.3 us, M = 8 6.2 / 12.0 / 13.0, against 10.6 / 16.1 /
    // 17.3 for the best tensor-memory kernel at either M): up to M = 8.  fp16 (9.7 / 17.3 / 17.7
    // against 11.1 / 19.1 / 19.3 us at M = 1) and W4A16 with smaller groups (CUDA-core kernels
    // whose time grows with M: behind from M = 2): a single row.
    SkGemvPlan pl;
    if (sk_gemv_plan(gemv_kind, q->M, q->N, q->K, num_sms, &pl)) {
      q->schedule = SK_SCHED_GEMV;
      return;
    }
  }
  const long long t256 = static_cast<long long>((q->M + 255) / 256) * ((q->N + 255) / 256);
  if (t256 >= num_sms) return;                       // large: hybrid (CTA pairs when eligible)
  // (W4A16 beyond 112 rows: the cluster schedule would need two narrower tiles per 128 weight
  // rows, i.e. dequantise every weight twice; Stream-K on whole-height tiles instead)
  if ((kernel_kind == 1 || (kernel_kind == 2 && (q->M <= 112 || !tiles_open))) && (q->K + 63) / 64 >= 8) {
    // Few tiles and a deep K: split every tile over the CTAs of a cluster.  Measured 15-25 %
    // ahead of Stream-K with either workspace fixup wherever it applies (at most half as many
    // tiles as SMs): the partials never leave the SMs and no flag is polled.
    sk_problem c = *q;
    c.schedule = SK_SCHED_CLUSTER;
    if (tiles_open && c.M > 64 && kernel_kind == 1) { c.tile_m = 128; c.tile_n = 128; }
    if (sk_make_sched(&c, kernel_kind, num_sms, nullptr, nullptr, nullptr) == SK_OK) {
      *q = c;
      return;
    }
  }
  if (q->M <= 64 && (tiles_open || (q->tile_m != 0 && q->tile_m != 128))) {
    // operands swapped: one tile per 128 weight rows
    const int tiles = (q->N + 127) / 128;
    // Whole tiles once they occupy half the SMs (measured, both kernels: a split tile's fix-up
    // costs more than the idle SMs: 16.0 against 17.7 us for W4A16 at 16 x 11008 x 4096),
    // Stream-K below that.
    q->schedule = 2 * tiles >= num_sms ? SK_SCHED_DP : SK_SCHED_STREAMK;
    if (q->schedule == SK_SCHED_DP && kernel_kind == 1 && tiles_open && q->layout == SK_LAYOUT_NT && tiles < num_sms) {
      // fewer weight rows per tile, so that (nearly) every SM gets a tile of its own: the weight
      // stream of one SM stays below ~50 GB/s, and 86 tiles of 128 rows leave 62 SMs idle
      // (measured at 16 x 11008 x 4096: 19.3 us with 138 tiles of 80 rows, 21.5 with 86 of 128)
      const int bm = ((q->N + num_sms - 1) / num_sms + 7) & ~7;
      if (bm >= 64 && bm < 128) {
        q->tile_m = (q->M + 15) & ~15;
        q->tile_n = bm;
      }
    }
    return;
  }
  if (kernel_kind == 1 && tiles_open && q->M > 128 && q->layout == SK_LAYOUT_NT && (num_sms & 1) == 0) {
    // More than one 128-row tile row: CTA pairs (256-row tiles, each CTA loading half of the
    // weight tile) halve the weight bytes every SM has to pull; whole tiles, width fitted so
    // that every pair gets one (multiples of 32 measured better than odd multiples of 16).
    // Measured 14-20 % ahead of single-CTA tiles at 256 x 11008, 256 x 12288, 512 x 4096.
    const int pairs = num_sms / 2;
    const int rows256 = (q->M + 255) / 256;
    if (rows256 <= pairs) {
      const int per_row = pairs / rows256;
      int bn = ((q->N + per_row - 1) / per_row + 31) & ~31;
      if (bn < 96) bn = 96;
      if (bn <= 256) {
        q->schedule = SK_SCHED_DP; q->tile_m = 256; q->tile_n = bn;
        return;
      }
    }
  }
  const int tiles_m = (q->M + 127) / 128;
  if (kernel_kind == 1 && tiles_open && tiles_m <= num_sms) {
    // widest column count per tile row that still gives every tile its own SM
    const int per_row = num_sms / tiles_m;
    int bn = ((q->N + per_row - 1) / per_row + 15) & ~15;
    // One tile row whose 128-wide tiles already occupy half the SMs: keep them (measured at
    // 128 x 11008 x 4096: 23.0 us with 86 tiles of 128, 22.9 with 115 of 96, 25.0 with 138 of
    // 80).
    if (tiles_m == 1 && bn < 128 && 2 * ((q->N + 127) / 128) >= num_sms) bn = 128;
    if (bn >= 80 && bn <= 256 && q->layout == SK_LAYOUT_NT) {
      q->schedule = SK_SCHED_DP; q->tile_m = 128; q->tile_n = bn;
      return;
    }
  }
  q->schedule = SK_SCHED_STREAMK;
  if (tiles_open && kernel_kind == 1) { q->tile_m = 128; q->tile_n = 128; }
}

int sk_make_sched(const sk_problem* p, int kernel_kind, int num_sms, sk_schedule_info* info,
                  SkSched* s, SkPlan* plan_out) {
  if (!p || num_sms <= 0) return SK_ERR_ARG;
  if (p->M <= 0 || p->N <= 0 || p->K <= 0) return SK_ERR_SHAPE;
  if (p->schedule == SK_SCHED_GEMV) {
    // the small-M CUDA-core path has no tiles to schedule: describe its grid
    if (kernel_kind == 3) kernel_kind = 1;
    if (kernel_kind == 1 && p->layout != SK_LAYOUT_NT) return SK_ERR_ARG;
    SkGemvPlan pl;
    if (!sk_gemv_plan(sk_gemv_kind(kernel_kind, p->flags), p->M, p->N, p->K, num_sms, &pl)) return SK_ERR_SHAPE;
    if (s) {
      memset(s, 0, sizeof(*s));
      s->grid = pl.grid;
    }
    if (plan_out) memset(plan_out, 0, sizeof(*plan_out));
    if (info) {
      memset(info, 0, sizeof(*info));
      info->tile_m = p->M; info->tile_n = pl.rows; info->tile_k = pl.k_per_split;
      info->tiles_m = 1; info->tiles_n = pl.groups; info->total_tiles = pl.groups;
      info->iters_per_tile = pl.splits;
      info->sk_tiles = pl.splits > 1 ? pl.groups : 0;
      info->dp_tiles = pl.splits > 1 ? 0 : pl.groups;
      info->grid = pl.grid;
      info->sk_iters_per_cta = 1;
      info->dp_waves = pl.splits > 1 ? 0 : 1;
      info->group_m = 1;
      info->swap_ab = 1;
    }
    return SK_OK;
  }
  SkPlan plan;
  int st = make_plan(p, kernel_kind, num_sms, &plan);
  if (st != SK_OK) return st;
  const int tr = kernel_kind == 0 ? 64 : kernel_kind == 3 ? 256 : plan.bm;   // tile rows (kernel space)
  const int tk = kernel_kind == 0 ? 16 : 64;
  const long long tiles_r = (plan.rows + tr - 1) / tr;
  const long long tiles_c = (plan.cols + plan.bn - 1) / plan.bn;
  const long long total = tiles_r * tiles_c;
  const long long I = (p->K + tk - 1) / tk;
  if (total > (1LL << 30)) return SK_ERR_LIMIT;
  const int P = num_sms;
  long long T;
  switch (p->schedule) {
    case SK_SCHED_STREAMK: T = total; break;
    case SK_SCHED_HYBRID:
    case SK_SCHED_HYBRID_DP_FIRST:
      // "Two-tile SK + DP": streamk_fp16.py:98-104
      T = total % P;
      if (total - T > P) T += P;
      break;
    case SK_SCHED_DP: T = 0; break;
    case SK_SCHED_CLUSTER: T = total; break;
    default: return SK_ERR_ARG;
  }
  const long long S = T * I;
  if (S >= (1LL << 31)) return SK_ERR_LIMIT;
  const long long dp = total - T;
  long long grid;
  if (dp > 0) grid = dp < P && T == 0 ? dp : P;
  else grid = S < P ? S : P;
  if (grid < 1) grid = 1;
  int split = 0;
  if (p->schedule == SK_SCHED_CLUSTER) {
    // the largest portable cluster that still gives every tile its own cluster in one wave
    if (kernel_kind != 1 && kernel_kind != 2) return SK_ERR_ARG;
    if (2 * total > P) return SK_ERR_SHAPE;
    // exchange buffers of wider tiles do not fit beside the ring
    if (plan.bn > (kernel_kind == 2 ? 112 : 192)) return SK_ERR_SHAPE;
    split = 2;
    while (split < 8 && 2 * split * total <= P) split *= 2;
    grid = total * split;
  }
  int gm = p->group_m;
  // Bands of sixteen tile rows: the tiles a wave of CTAs works on then share few row panels and
  // few column panels of the operands.  Measured on configuration 5 with the CTA-pair kernel
  // (one-pass ncu capture of dram__bytes): 3.19 GB of DRAM reads per product with bands of 8,
  // 2.98 with 12, 2.92 with 16 (algorithmic: 0.60 GB; L2 eviction-priority hints on the loads
  // changed nothing), and +0.8 % in the sustained loop.
  const int band = 16;
  if (gm <= 0) gm = (tiles_r > 1 && tiles_c > 1) ? (tiles_r < band ? static_cast<int>(tiles_r) : band) : 1;
  if (gm > tiles_r) gm = static_cast<int>(tiles_r);

  SkSched sc;
  sc.tiles_m = static_cast<int>(tiles_r);
  sc.tiles_n = static_cast<int>(tiles_c);
  sc.total_tiles = static_cast<int>(total);
  sc.iters_per_tile = static_cast<int>(I);
  sc.sk_tiles = static_cast<int>(T);
  sc.grid = static_cast<int>(grid);
  sc.sk_f = static_cast<int>(split ? I / split : S / grid);
  sc.sk_r = static_cast<int>(split ? I % split : S % grid);
  sc.split = split;
  sc.wide_base = -1;
  sc.dp_first = p->schedule == SK_SCHED_HYBRID_DP_FIRST ? 1 : 0;
  sc.group_m = gm;
  long long wide_units = 0;
  if (kernel_kind == 3 && p->schedule == SK_SCHED_HYBRID && p->tile_m == 0 && plan.bn == 256 &&
      (tiles_c & 1) == 0 && grid == P) {
    // CTA pairs, hybrid schedule, the library's own tile choice: the data-parallel part is
    // walked in units of two column-adjacent tiles that share every A stage (25 % fewer bytes
    // into an SM per flop).  As many full waves of such 256 x 512 units as fit are taken from
    // the front of the rasterised grid of units; the Stream-K part walks the halves of the
    // remaining units (sk_tile_mn, wide_base) — fewer tiles than the reference's two-tile rule
    // would give it, because a unit is two tiles.
    wide_units = tiles_r * (tiles_c / 2) / P * P;
    if (wide_units > 0) {
      const long long rest = total - 2 * wide_units;
      const long long Sw = rest * I;
      sc.tiles_n = static_cast<int>(tiles_c / 2);
      sc.total_tiles = static_cast<int>(rest);
      sc.sk_tiles = static_cast<int>(rest);
      sc.sk_f = static_cast<int>(Sw / P);
      sc.sk_r = static_cast<int>(Sw % P);
      sc.wide_base = static_cast<int>(wide_units);
      T = rest;
    }
  }
  sk_sched_finish(sc);
  if (s) *s = sc;
  if (plan_out) *plan_out = plan;
  if (info) {
    info->swap_ab = plan.swap;
    info->tile_m = plan.swap ? plan.bn : tr;
    info->tile_n = plan.swap ? tr : plan.bn;
    info->tile_k = tk;
    info->tiles_m = plan.swap ? sc.tiles_n : sc.tiles_m;
    info->tiles_n = plan.swap ? sc.tiles_m : static_cast<int>(tiles_c);
    info->total_tiles = static_cast<int>(total); info->iters_per_tile = sc.iters_per_tile;
    info->sk_tiles = sc.sk_tiles; info->dp_tiles = static_cast<int>(total - T);
    info->wide_units = static_cast<int>(wide_units);
    info->grid = sc.grid;
    info->sk_iters_per_cta = sc.sk_f; info->sk_iters_rem = sc.sk_r;
    info->dp_waves = wide_units ? static_cast<int>(wide_units / grid) : static_cast<int>((dp + grid - 1) / grid);
    info->dp_first = sc.dp_first;
    info->group_m = gm;
    info->cluster = split;
  }
  return SK_OK;
}

// CTA pairs pay off once the problem fills every pair with several 256 x 256 tiles; they
// are asked for explicitly with tile_m = 256.
static bool use_cta_pairs(const sk_problem* prob, int num_sms) {
  if (prob->layout != SK_LAYOUT_NT || (num_sms & 1) != 0) return false;
  if (prob->schedule == SK_SCHED_CLUSTER || prob->schedule == SK_SCHED_GEMV) return false;
  if (prob->tile_m == 256) return true;   // (tile_n: 0 = 256, or any multiple of 16 from 32; checked by the plan)
  if (prob->tile_m != 0 || prob->tile_n != 0) return false;
  const long long tiles = static_cast<long long>((prob->M + 255) / 256) * ((prob->N + 255) / 256);
  return tiles >= 2LL * (num_sms / 2);
}

void sk_f16_dispatch(const sk_problem* in, int num_sms, int n_peers, sk_problem* out, int* kernel_kind,
                     int* units) {
  *out = *in;
  // Fused all-gather: how the bytes to push compare with the mainloop (a GPU's stores reach
  // its peers at about 600 GB/s, its tensor cores do 1.3 PFLOP/s: 2167 K-steps' worth per peer).
  // From 60 % of the mainloop on, plain 256 x 256 tiles instead of the 256 x 512 units, whose
  // first results (and with them the transfer) would start twice as late; measured on 4 GPUs,
  // 8192 x 7168 x 8192 per GPU: 885 us against 966 with the units (the GEMM alone: 707 against
  // 655).  Beyond 100 % (the gather is link-bound) whole tiles only as well, because a split
  // tile reaches the peers at the very end of the kernel; measured on 8 GPUs, 8192 x 3584 x 8192
  // per GPU: 869 us with the units, 810 with hybrid 256 x 256 tiles, 780 data-parallel.
  if (n_peers > 0 && out->tile_m == 0 && 5LL * 2167 * n_peers > 3LL * in->K) {
    out->tile_m = 256;
    if (2167LL * n_peers > in->K && out->schedule == SK_SCHED_AUTO) out->schedule = SK_SCHED_DP;
  }
  sk_resolve_auto(out, 1, num_sms);
  // (the fused multi-GPU epilogues live in the CTA-pair kernel, not in the small-M path)
  if (n_peers != 0 && in->schedule == SK_SCHED_AUTO && out->schedule == SK_SCHED_GEMV) out->schedule = SK_SCHED_STREAMK;
  const bool pairs = use_cta_pairs(out, num_sms);
  *kernel_kind = pairs ? 3 : 1;
  *units = pairs ? num_sms / 2 : num_sms;
}

static int schedule_for(const sk_problem* p, int kernel_kind, int num_sms, int n_peers,
                        sk_schedule_info* out) {
  if (!out || !p) return SK_ERR_ARG;
  if (kernel_kind < 0 || kernel_kind > 3) return SK_ERR_ARG;
  sk_problem q = *p;
  if (kernel_kind == 1) {
    // exactly what sk_gemm_f16 would run: the pair kernel's schedule runs over pairs
    sk_f16_dispatch(p, num_sms, n_peers, &q, &kernel_kind, &num_sms);
  } else {
    sk_resolve_auto(&q, kernel_kind, num_sms);
  }
  const int st = sk_make_sched(&q, kernel_kind, num_sms, out, nullptr, nullptr);
  if (st == SK_OK) out->schedule = q.schedule;
  return st;
}

extern "C" int sk_schedule(const sk_problem* p, int kernel_kind, int num_sms,
                           sk_schedule_info* out) {
  return schedule_for(p, kernel_kind, num_sms, 0, out);
}

extern "C" int sk_schedule_gather(const sk_problem* p, int n_peers, int num_sms, sk_schedule_info* out) {
  if (n_peers < 0 || n_peers > SK_MAX_PEERS) return SK_ERR_ARG;
  return schedule_for(p, 1, num_sms, n_peers, out);
}

// Kernel-space schedule (rows = the 128-wide UMMA M side) from the logical description.
static SkSched sched_from_info(const sk_schedule_info* i) {
  SkSched s;
  s.tiles_m = i->swap_ab ? i->tiles_n : i->tiles_m;
  s.tiles_n = i->swap_ab ? i->tiles_m : i->tiles_n;
  s.total_tiles = i->total_tiles;
  s.iters_per_tile = i->iters_per_tile; s.sk_tiles = i->sk_tiles; s.grid = i->grid;
  s.sk_f = i->sk_iters_per_cta; s.sk_r = i->sk_iters_rem; s.dp_first = i->dp_first;
  s.group_m = i->group_m;
  s.split = i->cluster;
  s.wide_base = -1;
  if (i->wide_units > 0) {   // CTA pairs: the schedule's tiles are halves of units two tiles wide
    s.tiles_n = i->tiles_n / 2;
    s.total_tiles = i->sk_tiles;
    s.wide_base = i->wide_units;
  }
  sk_sched_finish(s);
  return s;
}

extern "C" int sk_cta_interval(const sk_schedule_info* info, int cta, int64_t* begin,
                               int64_t* end) {
  if (!info || !begin || !end || cta < 0 || cta >= info->grid) return SK_ERR_ARG;
  const SkSched s = sched_from_info(info);
  *begin = sk_cta_begin(s, cta);
  *end = sk_cta_begin(s, cta + 1);
  return SK_OK;
}

extern "C" int sk_tile_coords(const sk_schedule_info* info, int tile, int* tile_m, int* tile_n) {
  if (!info || !tile_m || !tile_n || tile < 0 || tile >= info->total_tiles) return SK_ERR_ARG;
  const SkSched s = sched_from_info(info);
  int r, c;
  sk_tile_mn(s, tile, r, c);
  *tile_m = info->swap_ab ? c : r;
  *tile_n = info->swap_ab ? r : c;
  return SK_OK;
}

extern "C" size_t sk_workspace_bytes(int num_sms) {
  if (num_sms <= 0) return 0;
  return sk_ws_total_bytes(num_sms);
}

extern "C" int sk_workspace_init(void* ws, size_t bytes, void* stream) {
  if (!ws) return SK_ERR_WORKSPACE;
  if (bytes < SK_WS_HEADER) return SK_ERR_WORKSPACE;
  cudaError_t e = cudaMemsetAsync(ws, 0, bytes, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return sk_set_cuda_error(e);
  return SK_OK;
}

extern "C" int sk_poll_status(const void* ws, sk_status* host_out, void* stream) {
  if (!ws || !host_out) return SK_ERR_ARG;
  cudaError_t e = cudaMemcpyAsync(host_out, ws, sizeof(sk_status), cudaMemcpyDeviceToHost,
                                  static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return sk_set_cuda_error(e);
  return SK_OK;
}

extern "C" int sk_memcpy2d_async(void* dst, size_t dst_pitch, const void* src, size_t src_pitch,
                                 size_t width_bytes, size_t rows, void* stream) {
  if (!dst || !src || width_bytes == 0 || rows == 0) return SK_ERR_ARG;
  if (dst_pitch < width_bytes || src_pitch < width_bytes) return SK_ERR_ARG;
  cudaError_t e = cudaMemcpy2DAsync(dst, dst_pitch, src, src_pitch, width_bytes, rows, cudaMemcpyDefault,
                                    static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return sk_set_cuda_error(e);
  return SK_OK;
}
