// W4A16 Stream-K GEMM on sm_100a: C[M,N] = A[M,K] . W^T, W = (q - z) * s with
// uint4 q, per-group (128 along K) uint4 zero-point z and fp16 scale s.
//
// Stands in for the TL kernel of streamk_fp16_ladder_block_reduce_q4.py:143-522
// (int8-packed weight tile in shared memory, decode_i4u_to_f16 in registers immediately
// ahead of the mma, …q4.py:255-294) and for its CPU weight preparation (LadderPermutate +
// LOP3Permutate, …q4.py:568-595).  The reference applies no scale or zero-point; with s = 1,
// z = 0 this kernel computes the same C = A . unpack_u4(qB)^T.
//
// Packed image (sk_prepack_q4):
//   nibble blocks  [n_block][k_block] of 128 rows x 64 K = 4096 B, stored as
//                  [half h][row r][16 B]; the 16 B hold K = h*32 .. h*32+31 of row r
//                  as four words, each word's eight nibbles in the order
//                  e0 e2 e4 e6 e1 e3 e5 e7 so that (w >> 4i) & 0x000F000F yields
//                  the fp16 pair (e(2i), e(2i+1)) in one lop3;
//   group blocks   [n_block][group] = 128 fp16 scales + 128 uint8 zero-points (384 B).
//
// Data path.  The weights ALWAYS feed the UMMA M dimension (128 weight rows per tile) and the
// activations the N dimension (a tile spans tile_m = 16 .. 128 rows of C; C is stored
// transposed).  That makes the weights the UMMA's A operand, which may live in tensor memory:
// a dequantise thread owns one weight row (TMEM lane), turns its packed words into halves in
// registers and writes them straight to tensor memory (tcgen05.st); the MMA issuer reads them
// from there (tcgen05.mma with the A operand in TMEM).  The dequantised weights never pass
// through shared memory: no swizzled stores, no generic-to-async proxy fence, and the shared
// memory holds nothing but the load ring (activation tile + packed block + group block per
// stage), which can therefore be deep.
//
// CTA roles (736 threads): warp 0 producer (TMA activation tile + bulk copies of the packed
// blocks), warp 1 MMA issuer, warps 2..5 epilogue, warps 6..21 dequantise in four groups of
// four (one warp per TMEM lane quadrant; group g takes stages g, g+4, ... whole), warp 22
// second MMA issuer (narrow tiles).  A stage is one scale group (128 of K, two K steps).
// Tensor memory (512 columns): [0, 256) the dequantised-weight ring, four slots of 64 columns
// (slot g belongs to group g); [256, 512) the accumulators (two buffers, each one or, with two
// issuers, two accumulators).
#include "sk_common.cuh"
#include "sk_epilogue.cuh"

namespace {

using namespace skptx;

constexpr int BM = SK_BM;
constexpr int BK = 64;
constexpr int Q_BLOCK_BYTES = 128 * BK / 2;    // 4096: packed nibbles of 128 weight rows x 64 K
constexpr int SZ_BLOCK_BYTES = 128 * 2 + 128;  // 384: fp16 scales + uint8 zero-points of a group
constexpr int SZ_SLOT_BYTES = 4 * SZ_BLOCK_BYTES;   // a stage (128 of K) spans at most four groups (group size 32)
constexpr int KG = 2;                          // K steps per stage = one scale group (128 along K)
constexpr int MAX_LS = 16;                     // load stages (activation tile + packed block)
constexpr int DQ_GROUPS = 4;                   // dequantise groups = slots of the TMEM weight ring
constexpr int DQ_GROUP_WARPS = 4;              // one warp per TMEM lane quadrant
constexpr int DQ_WARPS = DQ_GROUPS * DQ_GROUP_WARPS;
constexpr int DQ_THREADS = DQ_WARPS * 32;
constexpr int NUM_THREADS = 64 + SK_EPI_THREADS + DQ_THREADS + 32;   // + warp 22, the second MMA issuer
constexpr int MMA_B_WARP = 6 + DQ_WARPS;
constexpr int W_SLOT_COLS = KG * 32;           // TMEM columns of one dequantised stage (128 K halves, two per column)
constexpr int W_RING_COLS = DQ_GROUPS * W_SLOT_COLS;   // 256
constexpr int TMEM_COLS = 512;
constexpr int CTRL_BYTES = 512;
constexpr int SMEM_LIMIT = 232448;

struct Ctrl {
  uint64_t load_full[MAX_LS];
  uint64_t load_empty[MAX_LS];
  uint64_t w_full[DQ_GROUPS];
  uint64_t w_empty[DQ_GROUPS];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint64_t recv_full;      // SK_SCHED_CLUSTER: the partial tiles of the other CTAs have arrived
  uint32_t tmem_base;
  uint32_t abort;
  uint32_t bcast;
  uint32_t ok[2];
  SkPending pend[2];
};
static_assert(sizeof(Ctrl) <= CTRL_BYTES, "Ctrl must fit its reserved space");

// Eight uint4 values of one packed word -> eight fp16 (q - z) * s, in K order.
// zmagic = half2(1024 + z), s2 = half2(s, s).  The subtraction is exact and the
// product is rounded once, exactly like ((q.half() - z.half()) * s) on the CPU.
__device__ __forceinline__ uint4 dequant_word(uint32_t w, __half2 zmagic, __half2 s2) {
  constexpr uint32_t MASK = 0x000F000Fu;
  constexpr uint32_t MAGIC = 0x64006400u;  // fp16 1024.0 in both halves
  uint32_t t[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t sh = w >> (4 * i);
    // (sh & MASK) | MAGIC in one lop3 (truth table 0xEA = (a & b) | c)
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(t[i]) : "r"(sh), "r"(MASK), "r"(MAGIC));
  }
  uint32_t o[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __half2 x = *reinterpret_cast<const __half2*>(&t[i]);
    const __half2 y = __hmul2(__hsub2(x, zmagic), s2);
    o[i] = *reinterpret_cast<const uint32_t*>(&y);
  }
  return make_uint4(o[0], o[1], o[2], o[3]);
}

// Shared memory: [LS activation stages][LS packed blocks][LS group blocks][Ctrl][cluster
// receive buffer]; LS (a multiple of DQ_GROUPS, so that a load slot always belongs to the same
// dequantise group) is chosen per launch.  p.row_tx_bytes holds the bytes of one K step's
// activation tile (bn rows x 128 B).
// MODE as in the fp16 kernel: SK_EPI_ATOMIC, SK_EPI_BLOCK_REDUCE, SK_EPI_WHOLE (data-parallel
// schedule, no fixup code) or SK_MODE_CLUSTER; one instantiation each.
constexpr int SK_MODE_CLUSTER = 3;

template <int MODE>
__global__ void __launch_bounds__(NUM_THREADS, 1)
sk_gemm_w4a16_kernel(const __grid_constant__ CUtensorMap tmA, const uint8_t* __restrict__ qblocks,
                     const uint8_t* __restrict__ szblocks, __half* __restrict__ C, const SkParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw_addr);
  const int LS = p.stages;
  const int a_tile_bytes = p.row_tx_bytes;         // activation tile bytes of one K step
  const int a_stage_bytes = KG * a_tile_bytes;
  const int off_q = LS * a_stage_bytes;
  const int off_sz = off_q + LS * KG * Q_BLOCK_BYTES;
  const uint32_t sA = base;
  const uint32_t sQ = base + off_q;
  const uint32_t sSZ = base + off_sz;
  Ctrl* ctrl = reinterpret_cast<Ctrl*>(smem + off_sz + LS * SZ_SLOT_BYTES);
  // Group g of a row covers K halves [g << (5 + gshift), ...): gshift 0 / 1 / 2 for group sizes
  // 32 / 64 / 128, 30 for one group per row (per-channel scales).  Group blocks of a row block
  // are consecutive in the image (q_groups of them).
  const int gshift = p.q_gshift;
  volatile uint32_t* abort_flag = &ctrl->abort;

  // Outside the cluster schedule the warp index is computed so that the compiler knows it to
  // be warp-uniform (role branches then do not count as divergent, see elect_one).  The cluster
  // kernel keeps the plain form and single-lane issue loops: with the uniform form its
  // barrier.cluster start-up barrier never completed (hung, cause not found by reading; the
  // plain form is the one that has always run).
  constexpr bool clustered = MODE == SK_MODE_CLUSTER;
  const int warp = clustered ? static_cast<int>(threadIdx.x >> 5) : uniform_warp_idx();
  const int lane = threadIdx.x & 31;
  const int pid = blockIdx.x;
  const SkSched& s = p.sched;
  const int kblocks = s.iters_per_tile;  // K / 64
  const int groups = p.q_groups;         // group blocks per 128-row block: K / group size, or 1
  if (threadIdx.x == 0) {
    sk_trace(p, 0);
    griddep_launch_dependents();   // the next kernel of the stream may begin its own start-up
  }
  // Split-K inside a cluster (sk_epilogue.cuh): receive buffer behind the control block,
  // staging area in the load ring, which is idle by then.
  const uint32_t recv_base = smem_u32(ctrl) + CTRL_BYTES;

  // Start-up.  Kernel entry -> first load is pure latency on every problem this kernel sees,
  // so the work is spread: an epilogue warp (idle until the first tile is done) sets the
  // barriers up, one per lane, while the producer warp works out its first segment and asks L2
  // for that segment's first packed blocks; the producer then waits for nothing but the
  // barriers (named barrier BAR_PRODUCER), and the tensor-memory allocation runs beside the
  // first loads, awaited by everybody else (BAR_CONSUMERS).
  constexpr int BAR_PRODUCER = 2, BAR_CONSUMERS = 3;
  if (warp == 2) {
    if (lane < LS) {
      mbar_init(smem_u32(&ctrl->load_full[lane]), 1);
      // the stage's dequant warps + the MMA commit (+ the other issuer's "seen it", see below)
      mbar_init(smem_u32(&ctrl->load_empty[lane]), DQ_GROUP_WARPS + 1 + (p.acc_b_off ? 1 : 0));
    } else if (lane < LS + DQ_GROUPS) {
      const int i = lane - LS;
      mbar_init(smem_u32(&ctrl->w_full[i]), DQ_GROUP_WARPS);   // one arrival per dequant warp of the group
      mbar_init(smem_u32(&ctrl->w_empty[i]), p.acc_b_off ? 2 : 1);   // MMA commit (+ the other issuer)
    } else if (lane < LS + DQ_GROUPS + 2) {
      const int i = lane - LS - DQ_GROUPS;
      mbar_init(smem_u32(&ctrl->tmem_full[i]), p.acc_b_off ? 2 : 1);   // one arrival per MMA issuer
      mbar_init(smem_u32(&ctrl->tmem_empty[i]), 4);
    } else if (lane == LS + DQ_GROUPS + 2) {
      if (clustered) mbar_init(smem_u32(&ctrl->recv_full), 5);   // 4 epilogue warps + the byte count
      ctrl->abort = 0u;
      ctrl->bcast = 0u;
      ctrl->pend[0].tile = -1;
      ctrl->pend[1].tile = -1;
    }
    fence_mbar_init();
    fence_proxy_async_smem();
    __syncwarp();
    named_bar_arrive(BAR_PRODUCER, 64);       // the producer warp waits on it
    if (clustered && lane == LS + DQ_GROUPS + 2)
      mbar_arrive_expect_tx(smem_u32(&ctrl->recv_full),
                            static_cast<uint32_t>((s.split - 1) * p.cl_per) * SK_CL_QUAD_BYTES);
  }
  // The producer's first segment, and the L2 hint for its first packed blocks (L2 is the
  // coherence point, so nothing can go stale; with SK_FLAG_PDL this runs while the previous
  // kernel of the stream is still going).
  const bool solo = clustered ? lane == 0 : true;   // which lanes of the producer warp run its loop
  SkCursor pcur;
  SkSeg pseg;
  bool phave = false;
  int ptr = 0, ptc = 0;
  if (warp == 0 && solo) {
    sk_cursor_init(s, pid, pcur);
    phave = sk_next(s, pid, pcur, pseg);
    if (phave) {
      sk_tile_mn(s, pseg.tile, ptr, ptc);
      if (lane == 0) {
        prefetch_tensormap(&tmA);
        int n = pseg.k1 - pseg.k0;
        if (n > 12) n = 12;
        bulk_prefetch_l2(qblocks + (static_cast<size_t>(ptr) * kblocks + pseg.k0) * Q_BLOCK_BYTES,
                         static_cast<uint32_t>(n) * Q_BLOCK_BYTES);
      }
    }
  }
  uint32_t tmem_base = 0;
  if (warp == 0) {
    named_bar_sync(BAR_PRODUCER, 64);
  } else {
    if (warp == 1) {
      tmem_alloc(smem_u32(&ctrl->tmem_base), TMEM_COLS);
      tmem_relinquish();
    }
    tc_fence_before();
    named_bar_sync(BAR_CONSUMERS, NUM_THREADS - 32);
    tc_fence_after();
    tmem_base = *reinterpret_cast<volatile uint32_t*>(&ctrl->tmem_base);
  }
  const uint32_t tmem_acc = tmem_base + W_RING_COLS;   // accumulators behind the weight ring
  if (threadIdx.x == 0) sk_trace(p, 1);
  // global memory is the previous kernel's until it has completed (no-op without SK_FLAG_PDL)
  griddep_wait();

  if (warp == 0) {
    // ------------------------------------------------------------- producer
    // (whole warp, one elected lane issues: see the warp index above; single lane in the cluster kernel)
    if (solo) {
      const bool leader = clustered ? true : elect_one();
      bool traced = false;
      bool arrived = false;   // this thread's share of the cluster's start-up barrier
      bool first_seg = true;
      int ls = 0;
      uint32_t lph = 0;
      bool ok = true;
      for (; ok && phave; phave = sk_next(s, pid, pcur, pseg)) {
        if (!first_seg) sk_tile_mn(s, pseg.tile, ptr, ptc);   // (the first segment's are known already)
        first_seg = false;
        const int tr = ptr;
        const int a_row0 = ptc * p.bn;    // first activation row of the tile; tr = 128-row block of the weight
        for (int k = pseg.k0; k < pseg.k1;) {
          // A stage carries the K steps of one scale group (two, unless the segment starts
          // or ends inside the group): one barrier round trip, one packed copy, one group block.
          const int n = ((k & 1) || k + 1 >= pseg.k1) ? 1 : 2;
          const uint32_t full = smem_u32(&ctrl->load_full[ls]);
          if (!sk_wait_bar(smem_u32(&ctrl->load_empty[ls]), lph ^ 1u, abort_flag, p, ls, 0)) {
            ok = false;
            break;
          }
          // the group blocks the stage's K range touches: one (group size 128 or per-channel) up to four
          const int g0 = (2 * k) >> gshift, g1 = (2 * (k + n) - 1) >> gshift;
          const int sz_bytes = (g1 - g0 + 1) * SZ_BLOCK_BYTES;
          if (leader) {
            mbar_arrive_expect_tx(full, n * (a_tile_bytes + Q_BLOCK_BYTES) + sz_bytes);
            bulk_load_1d(sQ + ls * KG * Q_BLOCK_BYTES,
                         qblocks + (static_cast<size_t>(tr) * kblocks + k) * Q_BLOCK_BYTES,
                         n * Q_BLOCK_BYTES, full);
            bulk_load_1d(sSZ + ls * SZ_SLOT_BYTES,
                         szblocks + (static_cast<size_t>(tr) * groups + g0) * SZ_BLOCK_BYTES, sz_bytes, full);
            for (int j = 0; j < n; ++j)
              tma_load_2d(sA + ls * a_stage_bytes + j * a_tile_bytes, &tmA, full, (k + j) * BK, a_row0);
          }
          k += n;
          if (++ls == LS) {
            ls = 0; lph ^= 1u;
            // ring full for the first time: a good moment for this thread's share of the
            // cluster's start-up barrier.  Its arrival releases: it has met (at the named
            // barrier above) the warp that initialised the mbarrier the other CTAs will signal.
            if (clustered && !arrived) { cluster_arrive(); arrived = true; }
          }
          if (leader && !traced) { sk_trace(p, 2); traced = true; }
        }
      }
      if (clustered && !arrived) cluster_arrive();
    } else if (clustered) {
      cluster_arrive_relaxed();
    }
  } else if (warp == 1 || warp == MMA_B_WARP) {
    // ------------------------------------------------------------- MMA issuers
    // Issuing a UMMA costs its thread tens of nanoseconds whatever the tile width, and a stage
    // is eight of them.  With room in tensor memory for two accumulators per buffer
    // (p.acc_b_off), a second thread takes every other stage of a segment and accumulates on
    // its own; the epilogue adds the two.
    // The whole warp walks the schedule and waits on the barriers; one elected lane issues the
    // tcgen05 instructions and barrier arrivals (see elect_one).
    const uint32_t me = warp == 1 ? 0u : 1u;
    bool in_loop = me == 0u || p.acc_b_off != 0;
    bool leader;
    if constexpr (clustered) {
      leader = lane == 0;
      in_loop = in_loop && leader;
    } else {
      leader = in_loop && elect_one();
    }
    if (in_loop) {
      const bool dual = p.acc_b_off != 0;
      bool arrived = false;    // this thread's share of the cluster's start-up barrier
      SkCursor cur;
      sk_cursor_init(s, pid, cur);
      SkSeg seg;
      int ls = 0, g = 0;
      uint32_t lph = 0, wph = 0, nseg = 0;
      bool ok = true;
      const uint64_t desc_hi = umma_desc_sw128_hi(16, 1024);
      const uint32_t act_lo0 = umma_desc_lo(sA);
      const uint32_t act_tile16 = static_cast<uint32_t>(a_tile_bytes) >> 4;
      const uint32_t idesc = p.idesc;
      while (ok && sk_next(s, pid, cur, seg)) {
        const uint32_t buf = nseg & 1u;
        const uint32_t acc_ph = (nseg >> 1) & 1u;
        if (!sk_wait_bar(smem_u32(&ctrl->tmem_empty[buf]), acc_ph ^ 1u, abort_flag, p, 16 + buf, 1))
          break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_acc + buf * p.acc_stride + me * p.acc_b_off;
        uint32_t accumulate = 0u;   // this thread's first UMMA of the segment overwrites its accumulator
        uint32_t si = 0;            // stage number inside the segment
        for (int k = seg.k0; k < seg.k1; ++si) {
          const int n = ((k & 1) || k + 1 >= seg.k1) ? 1 : 2;
          // Both issuers watch every stage's barriers complete, in order: a parity wait only
          // tells a phase from its neighbours, so a thread that skipped the other's stages could
          // take a slot's previous use for the one it waits for.  For the same reason a slot
          // must not be reused before BOTH have seen its current use (else a lagging issuer
          // could find the barrier two phases on, which looks like "not yet"): the issuer that
          // skips a stage arrives on the slot's release barriers too.
          if (!sk_wait_bar(smem_u32(&ctrl->load_full[ls]), lph, abort_flag, p, 32 + ls, 1) ||
              !sk_wait_bar(smem_u32(&ctrl->w_full[g]), wph, abort_flag, p, 48 + g, 1)) {
            ok = false;
            break;
          }
          if (leader && me == 0u && nseg == 0 && si >= 8 && si < 10) sk_trace_clk(p, 12 + 2 * (si - 8));   // barriers seen
          if (!dual || (si & 1u) == me) {
            tc_fence_after();
            if (leader && nseg == 0 && k == seg.k0) sk_trace(p, 3);
            for (int j = 0; j < n; ++j) {
              const uint32_t b_lo = act_lo0 + (ls * KG + j) * act_tile16;          // activations: UMMA N side
              const uint32_t a_t = tmem_base + g * W_SLOT_COLS + j * 32;            // weights: A operand in TMEM
#pragma unroll
              for (int kk = 0; kk < BK / 16; ++kk) {
                if (leader) umma_f16_ts(d_tmem, a_t + kk * 8, desc_hi | (b_lo + kk * 2), idesc, accumulate);
                accumulate = 1u;
              }
            }
            if (leader) {
              umma_commit(smem_u32(&ctrl->load_empty[ls]));
              umma_commit(smem_u32(&ctrl->w_empty[g]));
            }
            if (clustered && !arrived) { cluster_arrive_relaxed(); arrived = true; }
          } else if (leader) {
            mbar_arrive(smem_u32(&ctrl->load_empty[ls]));
            mbar_arrive(smem_u32(&ctrl->w_empty[g]));
          }
          if (leader && me == 0u && nseg == 0 && si >= 8 && si < 10) sk_trace_clk(p, 13 + 2 * (si - 8));   // issued / skipped
          k += n;
          if (++ls == LS) { ls = 0; lph ^= 1u; }
          if (++g == DQ_GROUPS) { g = 0; wph ^= 1u; }
        }
        if (!ok) break;
        // (an issuer that issued nothing in this segment has nothing to wait for)
        if (leader) {
          if (accumulate) umma_commit(smem_u32(&ctrl->tmem_full[buf]));
          else mbar_arrive(smem_u32(&ctrl->tmem_full[buf]));
        }
        ++nseg;
      }
      if (leader && me == 0u) sk_trace(p, 4);
      if (clustered && !arrived) cluster_arrive_relaxed();
    } else if (clustered) {
      cluster_arrive_relaxed();
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------- epilogue
    if constexpr (clustered)   // (takes part in the cluster's start-up barrier on its own)
      sk_cluster_send(p, static_cast<int>(cluster_ctarank()), warp, lane, tmem_acc,
                      smem_u32(&ctrl->tmem_full[0]), sA, recv_base, smem_u32(&ctrl->recv_full),
                      abort_flag, sk_cta_begin(s, pid) % s.iters_per_tile,
                      sk_cta_begin(s, pid + 1) - sk_cta_begin(s, pid));
    else
      sk_epilogue_loop<MODE, 4, 1>(p, C, pid, 0, warp, lane, tmem_acc, smem_u32(&ctrl->tmem_full[0]),
                             smem_u32(&ctrl->tmem_empty[0]), &ctrl->bcast, abort_flag, ctrl->pend);
  } else {
    // ------------------------------------------------------------- dequantise
    // Group g (four warps, one per TMEM lane quadrant) takes stages g, g + 4, ... whole; a
    // thread owns weight row `row` of the tile: the packed words of its row in, 64 halves of
    // K per K step out, into the TMEM lane of that row.  Load slots (LS is a multiple of four)
    // and TMEM slots are thus always used by the same group, which sees every phase of their
    // barriers in order.  What a stage costs a group is mostly issue slots (about 250
    // instructions per thread), so four groups keep all four schedulers busy while the waits
    // of one are covered by the arithmetic of the others.
    const int dw = warp - 6;
    const int grp = dw >> 2;
    const int row = (warp & 3) * 32 + lane;
    const uint32_t t_row = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16) + grp * W_SLOT_COLS;
    SkCursor cur;
    sk_cursor_init(s, pid, cur);
    SkSeg seg;
    int ls = grp;                 // load slot of this group's next stage
    uint32_t lph = 0, wph = 0;
    uint32_t sidx = 0;            // running stage number
    bool dead = false;
    const bool tracer = grp == 0 && (warp & 3) == 0 && lane == 0;
    int own = 0;                  // stages this group has done (tracing only)
    if (clustered) cluster_arrive_relaxed();
    while (sk_next(s, pid, cur, seg)) {
      for (int k = seg.k0; k < seg.k1;) {
        const int n = ((k & 1) || k + 1 >= seg.k1) ? 1 : 2;
        if ((sidx & (DQ_GROUPS - 1)) == static_cast<uint32_t>(grp)) {
          if (!dead) {
            // (warp-uniform outcome: the tensor-memory stores below are warp-wide instructions)
            const bool got = sk_wait_bar(smem_u32(&ctrl->load_full[ls]), lph, abort_flag, p, 64 + ls, 3) &&
                             sk_wait_bar(smem_u32(&ctrl->w_empty[grp]), wph ^ 1u, abort_flag, p, 80 + grp, 3);
            if (!__all_sync(0xffffffffu, got)) dead = true;
          }
          if (tracer && own >= 2 && own < 4) sk_trace_clk(p, 8 + 2 * (own - 2));    // stage start (waits done)
          if (!dead) {
            tc_fence_after();     // the MMAs that read this slot's previous contents have retired
            const uint8_t* sz = smem + off_sz + ls * SZ_SLOT_BYTES;
            const int g0 = (2 * k) >> gshift;    // first group block of the stage (slot-relative index 0)
            __half2 s2, zmagic;
            int cur_blk = -1;
            for (int j = 0; j < n; ++j) {
              const uint8_t* q = smem + off_q + (ls * KG + j) * Q_BLOCK_BYTES + row * 16;
              const uint4 w0 = *reinterpret_cast<const uint4*>(q);          // K 0..31 of the step
              const uint4 w1 = *reinterpret_cast<const uint4*>(q + 2048);   // K 32..63
              const uint32_t words[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
              uint32_t v[32];
#pragma unroll
              for (int h = 0; h < 2; ++h) {
                const int blk = ((2 * (k + j) + h) >> gshift) - g0;   // group of this 32-wide half step
                if (blk != cur_blk) {   // (group size 128: once per stage)
                  cur_blk = blk;
                  const uint8_t* b = sz + blk * SZ_BLOCK_BYTES;
                  const __half sc = *reinterpret_cast<const __half*>(b + row * 2);
                  const uint32_t z = b[256 + row];
                  s2 = __half2half2(sc);
                  const uint32_t zm = 0x64006400u | z | (z << 16);
                  zmagic = *reinterpret_cast<const __half2*>(&zm);
                }
#pragma unroll
                for (int c = 4 * h; c < 4 * h + 4; ++c) {
                  const uint4 o = dequant_word(words[c], zmagic, s2);
                  v[4 * c + 0] = o.x; v[4 * c + 1] = o.y; v[4 * c + 2] = o.z; v[4 * c + 3] = o.w;
                }
              }
              tmem_st_32x32(t_row + j * 32, v);
            }
            tmem_st_wait();
            tc_fence_before();    // the stores are ordered before the arrival the MMA issuer acquires
          }
          __syncwarp();
          if (lane == 0) {
            mbar_arrive(smem_u32(&ctrl->w_full[grp]));
            mbar_arrive(smem_u32(&ctrl->load_empty[ls]));
          }
          if (tracer && own >= 2 && own < 4) sk_trace_clk(p, 9 + 2 * (own - 2));    // stage handed over
          ++own;
          wph ^= 1u;
          ls += DQ_GROUPS;
          if (ls >= LS) { ls -= LS; lph ^= 1u; }
        }
        ++sidx;
        k += n;
      }
    }
  }

  // ------------------------------------------------------------- teardown
  tc_fence_before();
  bool reduce_ok = true;
  if constexpr (clustered) {
    if (!(warp >= 2 && warp < 6)) cluster_wait();   // start-up barrier, second half
    __syncwarp();
    // the chunks of the other CTAs, and the epilogue warps' own one
    reduce_ok = sk_wait_bar(smem_u32(&ctrl->recv_full), 0u, abort_flag, p, 40, 3);
    // Final barrier: nobody leaves while a copy out of its staging area may be in flight.
    // Arrive now, wait after the reduction.
    cluster_arrive();
    if (threadIdx.x == 0) sk_trace(p, 6);
  } else {
    __syncthreads();
  }
  // The accumulators have been read: the tensor memory can go back while the rest reduces.
  if (warp == 1) {
    if (*abort_flag) {
      const unsigned long long t0 = globaltimer_ns();
      while (globaltimer_ns() - t0 < 200000ULL) __nanosleep(1000);
    }
    tc_fence_after();
    __syncwarp();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
  if constexpr (clustered) {
    if (reduce_ok)
      sk_cluster_reduce(p, C, pid >> s.split_log2, static_cast<int>(cluster_ctarank()), recv_base);
    cluster_wait();
  } else {
    // Block-reduce fixup: every thread of the CTA now helps to reduce this CTA's slices of
    // the split tiles it took part in.
    if constexpr (MODE == SK_EPI_BLOCK_REDUCE) sk_reduce_pending<true>(p, C, pid, 0, ctrl->pend, ctrl->ok);
  }
  if (threadIdx.x == 32) sk_trace(p, 7);
}

// ---------------------------------------------------------------- prepack / dequant
// One thread per output word.  Source nibble e of an 8-element group sits at bits 4e.
// groups: group blocks per row (K / group size, or 1); is_signed: the nibbles are two's-complement
// int4, stored here as q + 8 with zero-point 8 (the same (q - z) * s arithmetic, exactly).
__global__ void prepack_q4_kernel(const uint32_t* __restrict__ qw, const __half* __restrict__ scales,
                                  const uint8_t* __restrict__ zeros, int N, int K,
                                  uint32_t* __restrict__ qout, uint8_t* __restrict__ szout,
                                  int nblocks, int kblocks, int groups, int is_signed) {
  const int kwords = K / 8;
  const size_t total_words = static_cast<size_t>(nblocks) * kblocks * 1024;
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total_words;
       i += stride) {
    const size_t blk = i >> 10;
    const int in_blk = static_cast<int>(i & 1023);
    const int h = in_blk >> 9;
    const int r = (in_blk >> 2) & 127;
    const int j = in_blk & 3;
    const int nb = static_cast<int>(blk / kblocks);
    const int kb = static_cast<int>(blk - static_cast<size_t>(nb) * kblocks);
    const int n = nb * 128 + r;
    uint32_t out = 0u;
    if (n < N) {
      uint32_t w = qw[static_cast<size_t>(n) * kwords + kb * 8 + h * 4 + j];
      if (is_signed) w ^= 0x88888888u;   // two's complement -> offset binary, every nibble
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        out |= ((w >> (8 * t)) & 0xFu) << (4 * t);            // even elements 0,2,4,6
        out |= ((w >> (8 * t + 4)) & 0xFu) << (4 * (t + 4));  // odd elements 1,3,5,7
      }
    }
    qout[i] = out;
  }
  const size_t total_sz = static_cast<size_t>(nblocks) * groups * 128;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total_sz;
       i += stride) {
    const size_t gblk = i >> 7;
    const int r = static_cast<int>(i & 127);
    const int nb = static_cast<int>(gblk / groups);
    const int g = static_cast<int>(gblk - static_cast<size_t>(nb) * groups);
    const int n = nb * 128 + r;
    __half sc = __float2half(0.f);
    uint8_t z = 0;
    if (n < N) {
      sc = scales ? scales[static_cast<size_t>(n) * groups + g] : __float2half(1.f);
      z = is_signed ? 8 : zeros ? static_cast<uint8_t>(zeros[static_cast<size_t>(n) * groups + g] & 0xF) : 0;
    }
    uint8_t* dst = szout + gblk * SZ_BLOCK_BYTES;
    *reinterpret_cast<__half*>(dst + r * 2) = sc;
    dst[256 + r] = z;
  }
}

// One thread per packed word -> eight halves of W[n, k..k+7].
__global__ void dequant_q4_kernel(const uint32_t* __restrict__ qblocks,
                                  const uint8_t* __restrict__ szblocks, int N, int K,
                                  __half* __restrict__ W, int ldw, int kblocks, int groups, int gshift) {
  const size_t nb_used = (static_cast<size_t>(N) + 127) / 128;
  const size_t total_words = nb_used * kblocks * 1024;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total_words;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t blk = i >> 10;
    const int in_blk = static_cast<int>(i & 1023);
    const int h = in_blk >> 9;
    const int r = (in_blk >> 2) & 127;
    const int j = in_blk & 3;
    const int nb = static_cast<int>(blk / kblocks);
    const int kb = static_cast<int>(blk - static_cast<size_t>(nb) * kblocks);
    const int n = nb * 128 + r;
    if (n >= N) continue;
    const uint8_t* sz = szblocks + (static_cast<size_t>(nb) * groups + ((2 * kb + h) >> gshift)) * SZ_BLOCK_BYTES;
    const __half sc = *reinterpret_cast<const __half*>(sz + r * 2);
    const uint32_t z = sz[256 + r];
    const uint32_t zm = 0x64006400u | z | (z << 16);
    const uint4 o = dequant_word(qblocks[i], *reinterpret_cast<const __half2*>(&zm), __half2half2(sc));
    __half* dst = W + static_cast<size_t>(n) * ldw + kb * 64 + h * 32 + j * 8;
    if ((reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
      *reinterpret_cast<uint4*>(dst) = o;
    } else {
      const __half* hv = reinterpret_cast<const __half*>(&o);
#pragma unroll
      for (int e = 0; e < 8; ++e) dst[e] = hv[e];
    }
  }
}

inline int q4_nblocks(int N) { return (N + 255) / 256 * 2; }

}  // namespace

int sk_make_tmap_f16(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols,
                     uint64_t ld_elems, uint32_t box_cols, uint32_t box_rows);

// group_size 32, 64, 128, or K / 0 (one group per row: per-channel scales) -> gshift, groups per row
static bool q4_group(int K, int group_size, int* gshift, int* groups) {
  if (group_size == 0 || (group_size == K && K > 128)) { *gshift = 30; *groups = 1; return true; }
  if (group_size == 32) *gshift = 0;
  else if (group_size == 64) *gshift = 1;
  else if (group_size == 128) *gshift = 2;
  else return false;
  *groups = K / group_size;
  return true;
}

extern "C" size_t sk_q4_bytes_ex(int N, int K, int group_size) {
  int gshift, groups;
  if (N <= 0 || K <= 0 || (K % 128) != 0 || !q4_group(K, group_size, &gshift, &groups)) return 0;
  const size_t nb = q4_nblocks(N);
  return nb * (K / 64) * Q_BLOCK_BYTES + nb * groups * SZ_BLOCK_BYTES;
}

extern "C" size_t sk_q4_bytes(int N, int K) { return sk_q4_bytes_ex(N, K, 128); }

extern "C" int sk_prepack_q4_ex(const void* qweight, const void* scales, const void* zeros, int N,
                                int K, int group_size, int is_signed, void* out, size_t out_bytes,
                                void* stream) {
  if (!qweight || !out) return SK_ERR_ARG;
  int gshift, groups;
  if (N <= 0 || K <= 0 || (K % 128) != 0) return SK_ERR_SHAPE;
  if (!q4_group(K, group_size, &gshift, &groups)) return SK_ERR_ARG;
  if (is_signed && zeros) return SK_ERR_ARG;     // signed int4 is symmetric: W = q * s
  if (out_bytes < sk_q4_bytes_ex(N, K, group_size)) return SK_ERR_WORKSPACE;
  if ((reinterpret_cast<uintptr_t>(out) & 15u) || (reinterpret_cast<uintptr_t>(qweight) & 3u))
    return SK_ERR_ALIGN;
  const int nb = q4_nblocks(N), kb = K / 64;
  uint8_t* o = static_cast<uint8_t*>(out);
  uint8_t* sz = o + static_cast<size_t>(nb) * kb * Q_BLOCK_BYTES;
  const size_t total = static_cast<size_t>(nb) * kb * 1024;
  const int grid = static_cast<int>((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  prepack_q4_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint32_t*>(qweight), static_cast<const __half*>(scales),
      static_cast<const uint8_t*>(zeros), N, K, reinterpret_cast<uint32_t*>(o), sz, nb, kb, groups,
      is_signed ? 1 : 0);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return sk_set_cuda_error(e);
  return SK_OK;
}

extern "C" int sk_prepack_q4(const void* qweight, const void* scales, const void* zeros, int N,
                             int K, void* out, size_t out_bytes, void* stream) {
  return sk_prepack_q4_ex(qweight, scales, zeros, N, K, 128, 0, out, out_bytes, stream);
}

extern "C" int sk_dequant_q4(const void* packed, int N, int K, void* W, int ldw, void* stream) {
  return sk_dequant_q4_ex(packed, N, K, 128, W, ldw, stream);
}

extern "C" int sk_dequant_q4_ex(const void* packed, int N, int K, int group_size, void* W, int ldw,
                                void* stream) {
  if (!packed || !W) return SK_ERR_ARG;
  int gshift, groups;
  if (N <= 0 || K <= 0 || (K % 128) != 0 || ldw < K) return SK_ERR_SHAPE;
  if (!q4_group(K, group_size, &gshift, &groups)) return SK_ERR_ARG;
  if (reinterpret_cast<uintptr_t>(packed) & 15u) return SK_ERR_ALIGN;
  const int nb = q4_nblocks(N), kb = K / 64;
  const uint8_t* o = static_cast<const uint8_t*>(packed);
  const uint8_t* sz = o + static_cast<size_t>(nb) * kb * Q_BLOCK_BYTES;
  const size_t total = (static_cast<size_t>(N) + 127) / 128 * kb * 1024;
  const int grid = static_cast<int>((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  dequant_q4_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const uint32_t*>(o), sz, N, K, static_cast<__half*>(W), ldw, kb, groups, gshift);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return sk_set_cuda_error(e);
  return SK_OK;
}

extern "C" int sk_gemm_w4a16(const sk_problem* prob, const void* A, const void* packed, void* C,
                             void* ws, size_t ws_bytes, void* stream) {
  if (!prob || !A || !packed || !C) return SK_ERR_ARG;
  if (prob->fixup != SK_FIXUP_ATOMIC && prob->fixup != SK_FIXUP_BLOCK_REDUCE) return SK_ERR_ARG;
  int num_sms = 0, dev_sms = 0;
  int st = sk_resolve_grid(prob, &num_sms, &dev_sms);
  if (st != SK_OK) return st;
  sk_problem resolved = *prob;   // SK_SCHED_AUTO -> a concrete schedule and tile
  sk_resolve_auto(&resolved, 2, num_sms);
  prob = &resolved;
  const int M = prob->M, N = prob->N, K = prob->K;
  if (M <= 0 || N <= 0 || K <= 0 || (K % 128) != 0) return SK_ERR_SHAPE;
  if (prob->lda < K || prob->ldc < N) return SK_ERR_SHAPE;
  const int gcode = prob->flags & SK_FLAG_Q4_GROUP_MASK;
  const int group_size = gcode == SK_FLAG_Q4_GROUP_32 ? 32 : gcode == SK_FLAG_Q4_GROUP_64 ? 64
                       : gcode == SK_FLAG_Q4_PER_CHANNEL ? 0 : 128;
  int gshift = 2, groups = K / 128;
  if (!q4_group(K, group_size, &gshift, &groups)) return SK_ERR_ARG;
  if ((reinterpret_cast<uintptr_t>(A) & 15u) || (reinterpret_cast<uintptr_t>(packed) & 15u))
    return SK_ERR_ALIGN;
  if ((prob->lda & 7) != 0 || (reinterpret_cast<uintptr_t>(C) & 1u) != 0) return SK_ERR_ALIGN;
  if (!ws || ws_bytes < sk_ws_total_bytes(dev_sms)) return SK_ERR_WORKSPACE;
  if ((reinterpret_cast<uintptr_t>(ws) & 255u) != 0) return SK_ERR_ALIGN;

  SkParams p;
  memset(&p, 0, sizeof(p));
  SkPlan plan;
  st = sk_make_sched(prob, 2, num_sms, nullptr, &p.sched, &plan);
  if (st != SK_OK) return st;
  if (prob->schedule == SK_SCHED_GEMV) {   // small M: the CUDA-core path (sk_gemv.cu)
    const uint8_t* qb0 = static_cast<const uint8_t*>(packed);
    return sk_launch_gemv_q4(prob, A, qb0, qb0 + static_cast<size_t>(q4_nblocks(N)) * (K / 64) * Q_BLOCK_BYTES, C,
                             gshift, groups, sk_ws_carve(ws, dev_sms), num_sms, dev_sms, stream);
  }
  p.M = M; p.N = N; p.K = K;
  p.lda = prob->lda; p.ldb = 0; p.ldc = prob->ldc;
  p.rows = plan.rows; p.cols = plan.cols;
  p.transposed = plan.swap;
  p.unit_ctas = 1;
  p.bm = BM;
  p.fixup = prob->fixup;
  p.c_vec_ok = ((reinterpret_cast<uintptr_t>(C) & 15u) == 0 && (prob->ldc & 7) == 0) ? 1 : 0;
  p.drop_flag_cta = prob->test_drop_flag_cta - 1;
  p.timeout_ns = (prob->fixup_timeout_us > 0 ? static_cast<unsigned long long>(prob->fixup_timeout_us)
                                             : 2000000ULL) * 1000ULL;
  p.ws = sk_ws_carve(ws, dev_sms);
  p.trace = sk_trace_buffer();
  if (!plan.swap || plan.bm != BM || plan.bn > 128) return SK_ERR_ARG;   // (make_plan: always swapped, tile_m <= 128)
  // The activation tile feeds the UMMA N side: bn = tile_m rows of A per K step.
  const int a_tile_bytes = plan.bn * BK * 2;
  // Tensor memory: [0, 256) the dequantised-weight ring, [256, 512) two accumulator buffers.
  // Narrow tiles (<= 64 columns) leave room for two accumulators per buffer, one per MMA
  // issuer (issuing a UMMA costs its thread about the same whatever the width).
  p.bn = plan.bn;
  const int acc_cols = (plan.bn + 31) & ~31;
  const bool dual = acc_cols <= 64;
  p.acc_b_off = dual ? acc_cols : 0;
  p.acc_stride = dual ? 2 * acc_cols : acc_cols;
  p.tmem_cols = TMEM_COLS;
  p.kpair = 1;
  const int split = p.sched.split;   // SK_SCHED_CLUSTER: CTAs per tile
  const int recv_bytes = split ? sk_cluster_recv_bytes(plan.bn, split) : 0;
  p.cl_per = split ? sk_cluster_quads_per_cta(plan.bn, split) : 1;
  p.cl_per_div = sk_div_make(p.cl_per);
  // Shared memory is all load ring: activation tiles + packed block + group block per stage,
  // in a multiple of DQ_GROUPS stages (a slot then always belongs to the same dequantise group).
  const int budget = SMEM_LIMIT - 1024 - CTRL_BYTES - recv_bytes;
  const int load_stage = KG * (a_tile_bytes + Q_BLOCK_BYTES) + SZ_SLOT_BYTES;
  p.q_gshift = gshift;
  p.q_groups = groups;
  int ls = budget / load_stage / DQ_GROUPS * DQ_GROUPS;
  if (ls > MAX_LS) ls = MAX_LS;
  if (ls < DQ_GROUPS) return SK_ERR_SHAPE;
  p.stages = ls;
  p.w_stages = DQ_GROUPS;
  p.row_tx_bytes = a_tile_bytes;
  p.col_stage_bytes = a_tile_bytes;
  p.idesc = umma_idesc_f16(BM, plan.bn, 0);

  CUtensorMap tmA;
  st = sk_make_tmap_f16(&tmA, A, M, K, prob->lda, BK, plan.bn);
  if (st != SK_OK) return st;
  const int nb = q4_nblocks(N), kb = K / 64;
  const uint8_t* qb = static_cast<const uint8_t*>(packed);
  const uint8_t* sz = qb + static_cast<size_t>(nb) * kb * Q_BLOCK_BYTES;

  // the staging area of the cluster exchange lives in the load ring
  if (split && ls * load_stage < recv_bytes) return SK_ERR_SHAPE;
  const int smem_bytes = ls * load_stage + 1024 + CTRL_BYTES + recv_bytes;
  static SkPerDeviceOnce attrs;
  cudaError_t e = attrs.run([]() {
    cudaError_t r = cudaSuccess;
    const void* kernels[4] = {
        reinterpret_cast<const void*>(sk_gemm_w4a16_kernel<SK_EPI_ATOMIC>),
        reinterpret_cast<const void*>(sk_gemm_w4a16_kernel<SK_EPI_BLOCK_REDUCE>),
        reinterpret_cast<const void*>(sk_gemm_w4a16_kernel<SK_EPI_WHOLE>),
        reinterpret_cast<const void*>(sk_gemm_w4a16_kernel<SK_MODE_CLUSTER>)};
    for (int i = 0; i < 4 && r == cudaSuccess; ++i)
      r = cudaFuncSetAttribute(kernels[i], cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_LIMIT);
    return r;
  });
  if (e != cudaSuccess) return sk_set_cuda_error(e);
  const cudaStream_t cs = static_cast<cudaStream_t>(stream);
  __half* Ch = static_cast<__half*>(C);
  const bool pdl = (prob->flags & SK_FLAG_PDL) != 0;
  if (split)
    e = sk_launch(sk_gemm_w4a16_kernel<SK_MODE_CLUSTER>, p.sched.grid, NUM_THREADS, smem_bytes, cs, split, pdl,
                  tmA, qb, sz, Ch, p);
  else if (prob->schedule == SK_SCHED_DP)   // whole tiles only: no fixup code
    e = sk_launch(sk_gemm_w4a16_kernel<SK_EPI_WHOLE>, p.sched.grid, NUM_THREADS, smem_bytes, cs, 1, pdl,
                  tmA, qb, sz, Ch, p);
  else if (prob->fixup == SK_FIXUP_ATOMIC)
    e = sk_launch(sk_gemm_w4a16_kernel<SK_EPI_ATOMIC>, p.sched.grid, NUM_THREADS, smem_bytes, cs, 1, pdl,
                  tmA, qb, sz, Ch, p);
  else
    e = sk_launch(sk_gemm_w4a16_kernel<SK_EPI_BLOCK_REDUCE>, p.sched.grid, NUM_THREADS, smem_bytes, cs, 1, pdl,
                  tmA, qb, sz, Ch, p);
  if (e != cudaSuccess) return sk_set_cuda_error(e);
  return SK_OK;
}
