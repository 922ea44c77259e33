// Epilogue shared by the tensor-core kernels: TMEM accumulator -> fp16 C, or the
// cross-CTA fixup of a partial tile.
//
// Two fixups, both on fp32 partial sums (the reference adds fp16 halves straight
// into a pre-zeroed C with T.atomic_addx2, streamk_fp16.py:248-255):
//
//   atomic        every contributor red.global.add's its partial into the tile's
//                 zero-kept slot; the last one to arrive (a counter tells) folds the
//                 slot into C and zeroes it again.  Order of additions is not fixed.
//
//   block_reduce  every contributor stores its partial and raises a flag, without ever
//                 waiting.  After a CTA has finished all of its segments it returns to
//                 the (at most two) split tiles it took part in, waits with a time limit
//                 for the tile's other contributors, and reduces ITS SLICE of the tile:
//                 contributor j of n sums elements [j*L/n, (j+1)*L/n) over all partials
//                 in ascending CTA order and stores them to C.  The order is fixed, so
//                 the result is bitwise reproducible, and the reduction of a tile that is
//                 split n ways is spread over n SMs instead of serialised on its owner.
//                 Nothing waits while it still owes work to anyone, so there is no cycle.
//
// Slot layout (private): float4 index = (column / 4) * 128 + row, so a warp's 32 rows
// write 512 contiguous bytes per instruction.
#pragma once
#include "sk_common.cuh"

constexpr int SK_BM = 128;
constexpr int SK_EPI_THREADS = 128;
constexpr int SK_EPI_BAR_ID = 1;

// Bounded mbarrier wait.  On time-out the waiter raises the CTA-wide abort flag
// and records the barrier; every other wait in the CTA then returns false too.
__device__ __forceinline__ bool sk_wait_bar(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag,
                                            const SkParams& p, uint32_t bar_id, uint32_t role) {
  if (skptx::mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = skptx::globaltimer_ns();
  unsigned spins = 0;
  for (;;) {
    if (skptx::mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if ((++spins & 7u) == 0u) {
      if (skptx::globaltimer_ns() - t0 > p.timeout_ns) {
        *abort_flag = 1u;
        sk_report(p.ws.status, SK_ERR_PIPE_TIMEOUT, bar_id, role);
        return false;
      }
    }
  }
}

// fp32 -> the 16-bit result type: fp16, or bfloat16 when the problem carries SK_FLAG_BF16
// (p.out_bf16).  C is addressed as 16-bit words either way.
__device__ __forceinline__ uint32_t sk_pack2(float a, float b, int bf16) {
  uint32_t r;
  if (bf16) asm("cvt.rn.bf16x2.f32 %0, %2, %1;" : "=r"(r) : "f"(a), "f"(b));   // (first source -> upper half)
  else      asm("cvt.rn.f16x2.f32 %0, %2, %1;" : "=r"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ __half sk_cvt1(float a, int bf16) {
  const uint32_t r = sk_pack2(a, 0.f, bf16);
  return __ushort_as_half(static_cast<unsigned short>(r & 0xFFFFu));
}

// nv (<= NC) fp32 values of tile row `grow`, columns gcol0.. -> 16-bit C  (NC = 16 or 32)
template <int NC>
__device__ __forceinline__ void sk_store_cols(__half* __restrict__ C, const SkParams& p, int grow,
                                              int gcol0, int nv, const float (&v)[NC]) {
  if (p.transposed) {
    __half* dst = C + static_cast<size_t>(gcol0) * p.ldc + grow;
#pragma unroll
    for (int j = 0; j < NC; ++j)
      if (j < nv) dst[static_cast<size_t>(j) * p.ldc] = sk_cvt1(v[j], p.out_bf16);
    return;
  }
  __half* dst = C + static_cast<size_t>(grow) * p.ldc + gcol0;
  if (p.c_vec_ok && nv == NC) {
#pragma unroll
    for (int j = 0; j < NC / 8; ++j) {
      uint4 u;
      u.x = sk_pack2(v[8 * j + 0], v[8 * j + 1], p.out_bf16);
      u.y = sk_pack2(v[8 * j + 2], v[8 * j + 3], p.out_bf16);
      u.z = sk_pack2(v[8 * j + 4], v[8 * j + 5], p.out_bf16);
      u.w = sk_pack2(v[8 * j + 6], v[8 * j + 7], p.out_bf16);
      *reinterpret_cast<uint4*>(dst + 8 * j) = u;
    }
  } else {
#pragma unroll
    for (int j = 0; j < NC; ++j)
      if (j < nv) dst[j] = sk_cvt1(v[j], p.out_bf16);
  }
}
__device__ __forceinline__ void sk_store_chunk1(__half* __restrict__ C, const SkParams& p, int grow,
                                                int gcol0, int nv, const float (&v)[32]) {
  sk_store_cols<32>(C, p, grow, gcol0, nv, v);
}

// Four columns (gcol..gcol+3) of tile row `grow` -> 16-bit C
__device__ __forceinline__ void sk_store4(__half* __restrict__ C, const SkParams& p, int grow, int gcol,
                                          const float4& x) {
  const float v[4] = {x.x, x.y, x.z, x.w};
  if (p.transposed) {
#pragma unroll
    for (int e = 0; e < 4; ++e)
      if (gcol + e < p.cols) C[static_cast<size_t>(gcol + e) * p.ldc + grow] = sk_cvt1(v[e], p.out_bf16);
  } else {
    __half* dst = C + static_cast<size_t>(grow) * p.ldc + gcol;
    if (p.c_vec_ok && gcol + 4 <= p.cols) {
      uint2 u;
      u.x = sk_pack2(v[0], v[1], p.out_bf16);
      u.y = sk_pack2(v[2], v[3], p.out_bf16);
      *reinterpret_cast<uint2*>(dst) = u;
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e)
        if (gcol + e < p.cols) dst[e] = sk_cvt1(v[e], p.out_bf16);
    }
  }
}

// ... and, in the fused all-gather, to the same place of every peer GPU's matrix.  `peers` is a
// compile-time null in every kernel but the gathering one, where the loop disappears.
__device__ __forceinline__ void sk_store_chunk(__half* __restrict__ C, const SkParams& p, int grow,
                                               int gcol0, int nv, const float (&v)[32],
                                               const SkPeers* peers = nullptr) {
  sk_store_chunk1(C, p, grow, gcol0, nv, v);
  if (peers != nullptr)
    for (int i = 0; i < peers->n; ++i) sk_store_chunk1(static_cast<__half*>(peers->c[i]), p, grow, gcol0, nv, v);
}

// Fused all-gather, split tiles: the reducers store with a row stride (consecutive threads take
// consecutive rows: whole lines of the fp32 partials in, one 32- or 64-byte run per row out),
// which the local L2 absorbs but NVLink does not.  So they store locally only, and this copies
// what they stored from the local matrix to every peer in contiguous runs: one row per warp and
// pass, 8 bytes per lane.  Items are the reducers' (item = 128 * chunk + row, a chunk = QC quads
// of four columns) of this CTA's 128 rows starting at r0; [begin, end) is the range the calling
// threads reduced.
__device__ __forceinline__ void sk_copy_items_to_peers(const __half* C, const SkParams& p,
                                                       const SkPeers* peers, int r0, int c0,
                                                       int rows_valid, int quads_valid, int qc, int begin, int end,
                                                       int warp, int nwarps, int lane) {
  for (int r = warp; r < rows_valid; r += nwarps) {
    if (end - 1 - r < 0) continue;
    const int qlo = (begin - r > 0 ? (begin - r + SK_BM - 1) >> 7 : 0) * qc;
    int qhi = ((end - 1 - r) >> 7) * qc + qc - 1;
    if (qhi > quads_valid - 1) qhi = quads_valid - 1;
    const size_t row_off = static_cast<size_t>(r0 + r) * p.ldc + c0;
    for (int q = qlo + lane; q <= qhi; q += 32) {
      const size_t off = row_off + static_cast<size_t>(q) * 4;
      if (c0 + q * 4 + 4 <= p.cols) {
        const uint2 v = __ldcg(reinterpret_cast<const uint2*>(C + off));
        for (int i = 0; i < peers->n; ++i) *reinterpret_cast<uint2*>(static_cast<__half*>(peers->c[i]) + off) = v;
      } else {
        for (int e = 0; e < 4; ++e)
          if (c0 + q * 4 + e < p.cols) {
            const __half v = C[off + e];
            for (int i = 0; i < peers->n; ++i) static_cast<__half*>(peers->c[i])[off + e] = v;
          }
      }
    }
  }
}

struct SkPending {
  int tile;    // -1 = none
  int first, last;
};

// Sum one slice of a split tile over all of its partials, in ascending CTA order, and store
// it.  An item is one row of one chunk of QC quads (QC * 4 columns): the thread that takes it
// reads QC float4 per contributor (the slots are laid out [quad][row], so a warp's 32 rows
// read 512 contiguous bytes per instruction, at offsets that are immediates of one base
// address) and writes QC * 8 contiguous bytes of C, i.e. whole 32-byte sectors.  V contributors
// are fetched at once: QC * V loads in flight per thread; the loop is bound by L2 latency, not
// by arithmetic.  The code is kept small on purpose: it runs once per launch, from cold
// instruction caches.
template <int QC, int V>
__device__ __forceinline__ void sk_reduce_items_qv(const SkParams& p, __half* __restrict__ C,
                                                   int first, int last, int rank, int r0, int c0,
                                                   int rows_valid, int valid_cols, int begin, int end,
                                                   int tid, int nthreads) {
  for (int it = begin + tid; it < end; it += nthreads) {
    const int row = it & (SK_BM - 1), chunk = it >> 7;
    if (row >= rows_valid) continue;
    int nv = valid_cols - chunk * (QC * 4);
    if (nv > QC * 4) nv = QC * 4;
    float acc[QC * 4];
#pragma unroll
    for (int e = 0; e < QC * 4; ++e) acc[e] = 0.f;
    const size_t item0 = static_cast<size_t>(chunk * QC) * SK_BM + row;   // float4 index of the first quad
    for (int cta = first; cta <= last; cta += V) {
      float4 x[V][QC];
#pragma unroll
      for (int v = 0; v < V; ++v) {
        const int c = cta + v <= last ? cta + v : last;   // (a repeated fetch, not added)
        // partial of contributor c: the first one's tail slot, everybody else's head slot
        const float4* src = reinterpret_cast<const float4*>(
                                p.ws.part_slots +
                                static_cast<size_t>(2 * (c * p.unit_ctas + rank) + (c == first ? 1 : 0)) * SK_SLOT_FLOATS) +
                            item0;
        // (quads past the tile's last column hold stale values inside the slot; never stored)
#pragma unroll
        for (int q = 0; q < QC; ++q) x[v][q] = __ldcg(src + q * SK_BM);
      }
#pragma unroll
      for (int v = 0; v < V; ++v) {
        if (cta + v <= last) {
#pragma unroll
          for (int q = 0; q < QC; ++q) {
            acc[4 * q + 0] += x[v][q].x; acc[4 * q + 1] += x[v][q].y;
            acc[4 * q + 2] += x[v][q].z; acc[4 * q + 3] += x[v][q].w;
          }
        }
      }
    }
    sk_store_cols<QC * 4>(C, p, r0 + row, c0 + chunk * (QC * 4), nv, acc);
  }
}

// LIGHT: 16-column items (8 loads in flight instead of 16), for kernels with many threads and
// few registers each (the W4A16 kernel: 736 threads, 80 registers).
template <bool LIGHT = false>
__device__ __forceinline__ void sk_reduce_items(const SkParams& p, __half* __restrict__ C,
                                                const SkPending& pd, int pid, int rank, int tid,
                                                int nthreads, const SkPeers* peers) {
  constexpr int QC = LIGHT ? 4 : 8;
  const SkSched& s = p.sched;
  const int first = pd.first, last = pd.last;
  const int n = last - first + 1;
  int tr, tc;
  sk_tile_mn(s, pd.tile, tr, tc);
  const int r0 = (tr * p.unit_ctas + rank) * p.bm, c0 = tc * p.bn;
  int valid_cols = p.cols - c0;
  if (valid_cols > p.bn) valid_cols = p.bn;
  int rows_valid = p.rows - r0;
  if (rows_valid > p.bm) rows_valid = p.bm;
  const int L = ((valid_cols + QC * 4 - 1) / (QC * 4)) * SK_BM;  // items of this CTA's part of the tile
  const int j = pid - first;
  const int begin = j * L / n;
  const int end = (j + 1) * L / n;
  // The summation order (0 + p_first + p_first+1 + ...) is the same whatever the grouping.
  sk_reduce_items_qv<QC, 2>(p, C, first, last, rank, r0, c0, rows_valid, valid_cols, begin, end, tid, nthreads);
  if (peers != nullptr) {   // (called by every thread of the CTA, see sk_reduce_pending)
    __syncthreads();
    sk_copy_items_to_peers(C, p, peers, r0, c0, rows_valid, (valid_cols + 3) >> 2, QC, begin, end, tid >> 5,
                           nthreads >> 5, tid & 31);
  }
}

// Deferred block-reduce of the (at most two) split tiles this CTA took part in (see the
// header comment).  Called by EVERY thread of the CTA after all roles have finished;
// pend[0] is the tile the CTA started, pend[1] the tile it continued; ok[] is scratch.
template <bool LIGHT = false>
__device__ __forceinline__ void sk_reduce_pending(const SkParams& p, __half* __restrict__ C, int pid,
                                                  int rank, const SkPending* pend,
                                                  volatile uint32_t* ok, const SkPeers* peers = nullptr) {
  using namespace skptx;
  const int tid = threadIdx.x, nthreads = blockDim.x;
  if (pend[0].tile < 0 && pend[1].tile < 0) return;   // uniform over the CTA
  if (tid < 2) ok[tid] = 1u;
  __syncthreads();
  // 1. wait (bounded) for every contributor of both tiles; one flag per thread
  const int n0 = pend[0].tile >= 0 ? pend[0].last - pend[0].first + 1 : 0;
  const int n1 = pend[1].tile >= 0 ? pend[1].last - pend[1].first + 1 : 0;
  for (int i = tid; i < n0 + n1; i += nthreads) {
    const int t = i < n0 ? 0 : 1;
    const int k = i < n0 ? i : i - n0;
    const int first = pend[t].first;
    const int id = (first + k) * p.unit_ctas + rank;   // workspace index of that contributor
    const uint32_t* flag = (k == 0) ? (p.ws.flag_tail + id) : (p.ws.flag_head + id);
    if (!sk_wait_flag(flag, p.timeout_ns)) {
      sk_report(p.ws.status, SK_ERR_FIXUP_TIMEOUT, pend[t].tile, id);
      ok[t] = 0u;
    }
  }
  __syncthreads();
  if (tid == 0) sk_trace(p, 8);
  // 2. reduce this CTA's slice of each tile
  if (LIGHT && peers == nullptr && pend[0].tile >= 0 && pend[1].tile >= 0) {
    // Many threads, few items each (the W4A16 kernel: 736 threads for at most 512 items per
    // slice): the two tiles' slices side by side, half of the CTA each, instead of one after
    // the other -- half as many L2 round trips in a row.  (Which thread sums an element does
    // not change the order of its additions.)
    const int half = (nthreads >> 6) << 5;        // whole warps
    const int t = tid < half ? 0 : 1;
    if (ok[t] != 0u)
      sk_reduce_items<LIGHT>(p, C, pend[t], pid, rank, t ? tid - half : tid, t ? nthreads - half : half, peers);
    if (tid == 0) { sk_trace(p, 9); sk_trace(p, 10); }
  } else {
#pragma unroll
    for (int t = 0; t < 2; ++t) {
      if (pend[t].tile >= 0 && ok[t] != 0u) sk_reduce_items<LIGHT>(p, C, pend[t], pid, rank, tid, nthreads, peers);
      if (tid == 0) sk_trace(p, 9 + t);
    }
  }
  // 3. everybody has read what it needs; the last contributor to get here re-arms the flags
  __syncthreads();
  if (tid < 2 && pend[tid].tile >= 0) {
    const int first = pend[tid].first, last = pend[tid].last;
    const int uc = p.unit_ctas;
    const uint32_t old = atom_add_acqrel_u32(p.ws.done + first * uc + rank, 1u);
    if (old == static_cast<uint32_t>(last - first) && ok[tid] != 0u) {
      p.ws.flag_tail[first * uc + rank] = 0u;
      for (int peer = first + 1; peer <= last; ++peer) p.ws.flag_head[peer * uc + rank] = 0u;
      p.ws.done[first * uc + rank] = 0u;
    }
  }
  if (tid == 0) sk_trace(p, 11);
}

// Runs on the four epilogue warps (warps 2..5; `warp & 3` picks the TMEM lane quadrant a
// warp may read).  Leaves the split tiles still to be reduced in pend_out[0..1].  tmem_full_bar /
// tmem_empty_bar are the shared-memory addresses of two consecutive mbarriers each
// (one per accumulator).
// Does the segment [k0, k1) span at least two pipeline stages, i.e. did the second MMA issuer
// (if the kernel runs two, p.acc_b_off != 0) accumulate anything for it?
__device__ __forceinline__ bool sk_second_acc_used(const SkParams& p, int k0, int k1) {
  if (p.acc_b_off == 0) return false;
  const int len = k1 - k0;
  if (p.kpair) return (k0 & 1) ? len >= 2 : len >= 3;
  return len > p.kgroup;
}

// 32 accumulator columns of this thread's row; with b_off != 0 the sum of the two accumulators
// that two MMA-issuing threads filled (sk_gemm_f16.cu).
__device__ __forceinline__ void sk_load_acc(uint32_t taddr, uint32_t b_off, float (&v)[32]) {
  using namespace skptx;
  uint32_t r[32];
  tmem_ld_32x32(taddr, r);
  tmem_ld_wait();
#pragma unroll
  for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
  if (b_off != 0) {
    tmem_ld_32x32(taddr + b_off, r);
    tmem_ld_wait();
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] += __uint_as_float(r[j]);
  }
}

// MODE: which fixup code the instantiation carries.  SK_EPI_ANY decides at run time from
// p.fixup; SK_EPI_ATOMIC / SK_EPI_BLOCK_REDUCE carry one; SK_EPI_WHOLE none (data-parallel
// schedule: every segment is a whole tile).  Short kernels pay an instruction-cache miss for
// every line of code they touch, so their instantiations carry only what can run.
constexpr int SK_EPI_ANY = -1, SK_EPI_ATOMIC = SK_FIXUP_ATOMIC, SK_EPI_BLOCK_REDUCE = SK_FIXUP_BLOCK_REDUCE,
              SK_EPI_WHOLE = 2;

// Staging area of the TMA-store path: per epilogue warp buffers of 32 rows x 128 bytes (64
// fp16 columns, 128-byte swizzle), 1024-byte aligned; 32 KB in all: two buffers each for four
// epilogue warps, one each for eight.
constexpr int SK_CSTAGE_BYTES = 4 * 2 * 4096;

// Whole tile, 64 columns at a time: accumulator -> fp16 -> swizzled staging buffer -> one TMA
// store of a 64 x 32 box per warp (full 128-byte lines, issued asynchronously), instead of
// sixteen-byte stores to 32 different rows per instruction.  This warp takes the 64-column
// groups g_first, g_first + g_step, ... (the warps that share a TMEM lane quadrant split the
// columns).  NBUF: staging buffers per warp.  Returns the number of columns the warps handle
// together (a multiple of 64; the rest of the tile goes through sk_store_chunk).
template <int NBUF = 2>
__device__ __forceinline__ int sk_store_tile_tma(const SkParams& p, const CUtensorMap* tmC, uint32_t cstage,
                                                 int warp_slot, int lane, uint32_t t_addr, uint32_t b_off,
                                                 int grow0, int gcol0, int valid_cols, uint32_t& groups,
                                                 const SkPeers* peers = nullptr, int g_first = 0,
                                                 int g_step = 1) {
  using namespace skptx;
  const int full = valid_cols >> 6;
  for (int g = g_first; g < full; g += g_step, ++groups) {
    const uint32_t buf = cstage + static_cast<uint32_t>(warp_slot * NBUF + (NBUF == 2 ? (groups & 1u) : 0u)) * 4096u;
    // the store issued from this buffer NBUF groups ago must have read it
    if (lane == 0) tma_store_wait_read<NBUF - 1>();
    __syncwarp();
    // both 32-column reads of the group in flight before the one wait
    uint32_t raw[2][32];
    tmem_ld_32x32(t_addr + g * 64, raw[0]);
    tmem_ld_32x32(t_addr + g * 64 + 32, raw[1]);
    tmem_ld_wait();
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float v[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(raw[h][j]);
      if (b_off != 0) {   // second accumulator of a kernel with two MMA issuers
        uint32_t r2[32];
        tmem_ld_32x32(t_addr + b_off + g * 64 + h * 32, r2);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] += __uint_as_float(r2[j]);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t h0 = sk_pack2(v[8 * j + 0], v[8 * j + 1], p.out_bf16);
        const uint32_t h1 = sk_pack2(v[8 * j + 2], v[8 * j + 3], p.out_bf16);
        const uint32_t h2 = sk_pack2(v[8 * j + 4], v[8 * j + 5], p.out_bf16);
        const uint32_t h3 = sk_pack2(v[8 * j + 6], v[8 * j + 7], p.out_bf16);
        const uint32_t chunk = static_cast<uint32_t>(h * 4 + j);   // 16-byte chunk of the 128-byte row
        const uint32_t a = buf + static_cast<uint32_t>(lane) * 128u + ((chunk ^ (static_cast<uint32_t>(lane) & 7u)) << 4);
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(a), "r"(h0), "r"(h1), "r"(h2), "r"(h3)
                     : "memory");
      }
    }
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
      tma_store_2d(tmC, buf, gcol0 + g * 64, grow0);
      if (peers != nullptr)   // the same box into every peer's matrix, in the same bulk group
        for (int i = 0; i < peers->n; ++i) tma_store_2d(&peers->tm[i], buf, gcol0 + g * 64, grow0);
      tma_store_commit();
    }
  }
  return full * 64;
}

// EPI_WARPS: 4 (warps 2..5) or 8 (warps 2..9).  TMEM lets a warp read only the lane quadrant
// `warp & 3`, so with eight warps two share each quadrant and split a tile's columns: warp w
// takes the 64-column groups (and 32-column chunks) of parity (w - 2) / 4.
// Fused reduce-scatter: a whole tile leaves as fp32, 32 columns at a time: accumulator ->
// swizzled staging buffer (32 rows x 128 bytes) -> one TMA store of a 32 x 32 fp32 box into the
// receive slot `tm` of the tile's column block (x0 = the tile's first column inside that block).
// Ragged edges are clipped by the tensor map, so there is no register path.  One staging buffer
// per warp; this warp takes the groups g_first, g_first + g_step, ...
__device__ __forceinline__ void sk_store_tile_tma_f32(const CUtensorMap* tm, uint32_t cstage, int warp_slot,
                                                      int lane, uint32_t t_addr, int grow0, int x0,
                                                      int valid_cols, int g_first, int g_step) {
  using namespace skptx;
  const int ngroups = (valid_cols + 31) >> 5;
  const uint32_t buf = cstage + static_cast<uint32_t>(warp_slot) * 4096u;
  for (int g = g_first; g < ngroups; g += g_step) {
    if (lane == 0) tma_store_wait_read<0>();   // the previous store from this buffer has read it
    __syncwarp();
    uint32_t raw[32];
    tmem_ld_32x32(t_addr + g * 32, raw);
    tmem_ld_wait();
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const uint32_t a = buf + static_cast<uint32_t>(lane) * 128u + ((static_cast<uint32_t>(j) ^ (static_cast<uint32_t>(lane) & 7u)) << 4);
      asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(a), "r"(raw[4 * j]), "r"(raw[4 * j + 1]),
                   "r"(raw[4 * j + 2]), "r"(raw[4 * j + 3])
                   : "memory");
    }
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
      tma_store_2d(tm, buf, x0 + g * 32, grow0);
      tma_store_commit();
    }
  }
}

// FOLD: items the atomic fixup's last arriver fetches per thread and pass (2 = 16 loads in
// flight; 1 for kernels whose threads have few registers).
template <int MODE = SK_EPI_ANY, int EPI_WARPS = 4, int FOLD = (EPI_WARPS == 4 ? 2 : 1)>
__device__ __forceinline__ void sk_epilogue_loop(const SkParams& p, __half* __restrict__ C, int pid,
                                                 int rank, int warp, int lane, uint32_t tmem_base,
                                                 uint32_t tmem_full_bar, uint32_t tmem_empty_bar,
                                                 volatile uint32_t* bcast,
                                                 volatile uint32_t* abort_flag,
                                                 SkPending* pend_out,
                                                 const CUtensorMap* tmC = nullptr, uint32_t cstage = 0,
                                                 uint32_t* nseg_out = nullptr, const SkPeers* peers = nullptr) {
  using namespace skptx;
  constexpr int BM = SK_BM;
  constexpr int EPI_THREADS = 32 * EPI_WARPS;
  constexpr int EPI_BAR_ID = SK_EPI_BAR_ID;
  constexpr int NSUB = EPI_WARPS / 4;       // warps per TMEM lane quadrant
  constexpr int NBUF = EPI_WARPS == 4 ? 2 : 1;   // staging buffers per warp (sk_store_tile_tma)
  const SkSched& s = p.sched;
  const int q = warp & 3;            // TMEM lane quadrant this warp may read
  const int row = q * 32 + lane;     // row inside the tile
  const int sub = (warp - 2) >> 2;   // which of the quadrant's warps this is
  const int etid = (warp - 2) * 32 + lane;
  SkCursor cur;
  sk_cursor_init(s, pid, cur);
  SkSeg seg;
  uint32_t nseg = 0;
  uint32_t tma_groups = 0;   // TMA store groups this warp has issued
  bool dead = false;
  SkPending head{-1, 0, 0}, tail{-1, 0, 0};
  while (sk_next(s, pid, cur, seg)) {
    const uint32_t buf = nseg & 1u;
    const uint32_t acc_ph = (nseg >> 1) & 1u;
    ++nseg;
    int tr, tc;
    sk_tile_mn(s, seg.tile, tr, tc);
    const int r0 = (tr * p.unit_ctas + rank) * p.bm, c0 = tc * p.bn;
    const int grow = r0 + row;
    const bool row_ok = row < p.bm && grow < p.rows;   // (rows past the tile pitch hold stale data)
    const bool warp_ok = q * 32 < p.bm && (r0 + q * 32) < p.rows;  // warp-uniform
    int valid_cols = p.cols - c0;
    if (valid_cols > p.bn) valid_cols = p.bn;
    const int nchunks = (valid_cols + 31) >> 5;
    const bool whole = MODE == SK_EPI_WHOLE || (seg.k0 == 0 && seg.k1 == s.iters_per_tile);
    const bool atomic = MODE == SK_EPI_ATOMIC || (MODE == SK_EPI_ANY && p.fixup == SK_FIXUP_ATOMIC);
    int first = 0, last = 0;
    if (!whole) sk_tile_ctas(s, seg.tile, first, last);
    const bool is_tail = !whole && seg.k0 == 0;   // this CTA starts the tile (its "owner")

    // A wait that ran out must not leave the warps disagreeing: every epilogue
    // thread keeps walking the segment list (and meeting the named barriers) but
    // stops touching tensor memory.
    if (!dead) {
      const bool got = sk_wait_bar(tmem_full_bar + 8u * buf, acc_ph, abort_flag, p, 24 + buf, 2);
      if (!__all_sync(0xffffffffu, got)) dead = true;
    }
    tc_fence_after();
    if (nseg == 1 && etid == 0) sk_trace(p, 5);
    const uint32_t t_addr = tmem_base + buf * p.acc_stride + (static_cast<uint32_t>(q * 32) << 16);

    const int me = pid * p.unit_ctas + rank;             // workspace index of this CTA
    const int first_id = first * p.unit_ctas + rank;     // ... of the tile's first contributor
    float* acc_slot = p.ws.acc_slots + static_cast<size_t>(first_id) * SK_SLOT_FLOATS;
    float* my_part = p.ws.part_slots + static_cast<size_t>(2 * me + (is_tail ? 1 : 0)) * SK_SLOT_FLOATS;

    // two MMA issuers: the second one's accumulator holds every other stage of the segment
    const bool two = sk_second_acc_used(p, seg.k0, seg.k1);
    int c_first = 0;   // first 32-column chunk that still has to go through the register path
    if (whole && p.c_tma && cstage != 0 && warp_ok && !dead)
      c_first = sk_store_tile_tma<NBUF>(p, tmC, cstage, warp - 2, lane, t_addr, two ? p.acc_b_off : 0,
                                        r0 + q * 32, c0, valid_cols, tma_groups, peers, sub, NSUB) >> 5;
    if (warp_ok && !dead) {
      for (int c = c_first + sub; c < nchunks; c += NSUB) {
        float v[32];
        sk_load_acc(t_addr + c * 32, two ? p.acc_b_off : 0, v);
        if (!row_ok) continue;
        int nv = valid_cols - c * 32;
        if (nv > 32) nv = 32;
        if (whole) {
          sk_store_chunk(C, p, grow, c0 + c * 32, nv, v, peers);
        } else if (atomic) {
#pragma unroll
          for (int j = 0; j < 8; ++j)
            if (4 * j < nv)
              red_add_v4(acc_slot + (static_cast<size_t>(c * 8 + j) * BM + row) * 4, v[4 * j],
                         v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j)
            if (4 * j < nv)
              __stcg(reinterpret_cast<float4*>(my_part + (static_cast<size_t>(c * 8 + j) * BM + row) * 4),
                     make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]));
        }
      }
    }
    // hand the accumulator back to the MMA warp
    tc_fence_before();
    __syncwarp();
    if (lane == 0) {
      // with CTA pairs the barrier lives in the leader CTA (a shared::cluster address)
      if (p.unit_ctas == 2) mbar_arrive_cluster(tmem_empty_bar + 8u * buf);
      else mbar_arrive(tmem_empty_bar + 8u * buf);
    }

    if (whole) continue;
    if (atomic) {
      __threadfence();
      named_bar_sync(EPI_BAR_ID, EPI_THREADS);
      if (etid == 0) {
        const uint32_t old = atom_add_acqrel_u32(p.ws.counters + first_id, 1u);
        *bcast = (old == static_cast<uint32_t>(last - first)) ? 1u : 0u;
      }
      named_bar_sync(EPI_BAR_ID, EPI_THREADS);
      if (*bcast != 0u) {
        // last contributor: fold the slot into C and leave the slot zeroed; all 128
        // threads share the work whatever the number of valid rows
        __threadfence();
        int rows_valid = p.rows - r0;
        if (rows_valid > p.bm) rows_valid = p.bm;
        const int L = ((valid_cols + 31) >> 5) * BM;   // items: one row of one 32-column chunk
        float4* slot4 = reinterpret_cast<float4*>(acc_slot);
        const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
        // FOLD items (row x 32-column chunk) per thread and pass: 8 loads in flight each, the pass is
        // bound by L2 latency
        for (int it = etid; it < L; it += FOLD * EPI_THREADS) {
          float4 x[FOLD][8];
          float4* src[FOLD];
          bool on[FOLD];
#pragma unroll
          for (int h = 0; h < FOLD; ++h) {
            const int i = it + h * EPI_THREADS;
            on[h] = i < L && (i & (BM - 1)) < rows_valid;
            src[h] = slot4 + static_cast<size_t>((i >> 7) * 8) * BM + (i & (BM - 1));
            if (on[h]) {
#pragma unroll
              for (int qd = 0; qd < 8; ++qd) x[h][qd] = __ldcg(src[h] + qd * BM);
            }
          }
#pragma unroll
          for (int h = 0; h < FOLD; ++h) {
            if (!on[h]) continue;
            const int i = it + h * EPI_THREADS;
            int nv = valid_cols - (i >> 7) * 32;
            if (nv > 32) nv = 32;
            float v[32];
#pragma unroll
            for (int qd = 0; qd < 8; ++qd) {
              __stcg(src[h] + qd * BM, zero);
              v[4 * qd + 0] = x[h][qd].x; v[4 * qd + 1] = x[h][qd].y;
              v[4 * qd + 2] = x[h][qd].z; v[4 * qd + 3] = x[h][qd].w;
            }
            sk_store_cols<32>(C, p, r0 + (i & (BM - 1)), c0 + (i >> 7) * 32, nv, v);
          }
        }
        if (peers != nullptr) {
          named_bar_sync(EPI_BAR_ID, EPI_THREADS);
          sk_copy_items_to_peers(C, p, peers, r0, c0, rows_valid, (valid_cols + 3) >> 2, 8, 0, L, warp - 2,
                                 EPI_WARPS, lane);
        }
        if (etid == 0) p.ws.counters[first_id] = 0u;
      }
      named_bar_sync(EPI_BAR_ID, EPI_THREADS);  // bcast is reused by the next segment
    } else {
      // publish the partial; never wait here
      __threadfence();
      named_bar_sync(EPI_BAR_ID, EPI_THREADS);
      if (etid == 0 && me != p.drop_flag_cta)
        st_release_u32(is_tail ? (p.ws.flag_tail + me) : (p.ws.flag_head + me), 1u);
      SkPending& pd = is_tail ? tail : head;
      pd.tile = seg.tile; pd.first = first; pd.last = last;
    }
  }
  // the staging buffers must outlive the stores that read them
  if (p.c_tma && cstage != 0 && lane == 0) tma_store_wait_read<0>();
  if (nseg_out) *nseg_out = nseg;   // (a caller that goes on using the accumulator buffers)
  if (etid == 0) {
    sk_trace(p, 6);
    pend_out[0] = tail;   // reduced by the whole CTA once every role is done
    pend_out[1] = head;
  }
}

// ---------------------------------------------------------------------------------------
// SK_SCHED_CLUSTER: the CTAs of one thread-block cluster each hold a partial sum of the
// SAME tile (sk_sched.h, `split`).  The partials meet in distributed shared memory instead
// of the global workspace.  The tile's float4 column groups ("quads", 4 columns x 128 rows)
// are dealt out in runs of `per` to the cluster's CTAs.  A CTA
//   1. copies its accumulator from tensor memory into a staging area (the operand ring,
//      idle by then), one contiguous chunk per destination CTA, its own chunk straight into
//      its receive buffer;
//   2. sends every other chunk with one bulk shared-to-shared copy, whose bytes are counted
//      on an mbarrier of the destination;
//   3. waits (bounded) on its own mbarrier for the S-1 chunks addressed to it, sums its quads
//      over the senders in CTA order (bitwise reproducible) and writes them to C.
// Two cluster barriers frame this: one at start-up (nobody writes into a CTA before its
// mbarrier exists; its arrivals are spread over the start of the mainloop, where they cost
// nothing) and one at the end (nobody leaves while its outgoing copies may still be read from
// its staging area; its latency overlaps step 3's arithmetic).
//
// Chunk layout, same in the staging area and in a receive slot: quad q of the chunk starts
// at q * SK_CL_QUAD_BYTES, row r of it 16*r bytes further.  The 16 bytes of padding per quad
// let a quarter warp read one row of eight quads without a bank conflict.  A receive buffer
// is S such chunks, indexed by sender.
// ---------------------------------------------------------------------------------------
constexpr int SK_CL_QUAD_BYTES = SK_BM * 16 + 16;

__host__ __device__ __forceinline__ int sk_cluster_quads_per_cta(int bn, int split) {
  return ((bn >> 2) + split - 1) / split;
}
// bytes of a receive buffer, and of the staging area
__host__ __device__ __forceinline__ int sk_cluster_recv_bytes(int bn, int split) {
  return split * sk_cluster_quads_per_cta(bn, split) * SK_CL_QUAD_BYTES;
}

// Steps 1 and 2; runs on the four epilogue warps.  k_begin, k_iters: this CTA's range of K
// iterations (an empty one contributes zeros).  recv_bar: this CTA's mbarrier, initialised with
// five arrivals (one per epilogue warp here, one with the expected byte count).
// Chunks are sent as soon as they are staged, so one travels while the next is being staged.
__device__ __forceinline__ void sk_cluster_send(const SkParams& p, int rank, int warp, int lane,
                                                uint32_t tmem_base, uint32_t tmem_full_bar,
                                                uint32_t stage_base, uint32_t recv_base,
                                                uint32_t recv_bar, volatile uint32_t* abort_flag,
                                                int k_begin, int k_iters) {
  using namespace skptx;
  const int S = p.sched.split;
  const int q = warp & 3;
  const int per = p.cl_per;
  const uint32_t chunk_bytes = static_cast<uint32_t>(per) * SK_CL_QUAD_BYTES;
  const uint32_t row_off = static_cast<uint32_t>(q * 32 + lane) * 16u;
  const bool has_work = k_iters > 0;
  bool live = has_work;
  cluster_arrive_relaxed();   // start-up barrier of the cluster, first half
  if (has_work) {
    const bool got = sk_wait_bar(tmem_full_bar, 0u, abort_flag, p, 24, 2);
    if (!__all_sync(0xffffffffu, got)) live = false;
  }
  tc_fence_after();
  if (warp == 2 && lane == 0) sk_trace(p, 5);
  cluster_wait();             // second half: every CTA's mbarrier exists
  const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
  // two MMA issuers: the second accumulator is in use if the CTA's K range has a second stage
  const uint32_t b_off = sk_second_acc_used(p, k_begin, k_begin + k_iters) ? static_cast<uint32_t>(p.acc_b_off) : 0u;
  if (per >= 8) {
    // Wide chunks (a 32-column read never spans two of them): one chunk after the other,
    // starting with the next CTA's, so that the senders do not all aim at the same
    // destination at once (measured: 0.9 us on a 128 x 128 tile split four ways); the CTA's
    // own chunk comes last and goes straight into its receive buffer.
    const int Q = p.bn >> 2;
    for (int i = 1; i <= S; ++i) {
      int owner = rank + i;
      if (owner >= S) owner -= S;
      const bool mine = owner == rank;
      const int q0 = owner * per;
      int q1 = q0 + per;
      if (q1 > Q) q1 = Q;
      const uint32_t dst0 =
          (mine ? recv_base : stage_base) + static_cast<uint32_t>(owner) * chunk_bytes + row_off;
      for (int qq = q0; qq < q1; qq += 8) {
        float v[32];
        if (live) {
          sk_load_acc(t_addr + 4 * qq, b_off, v);
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = 0.f;
        }
        const uint32_t dst = dst0 + static_cast<uint32_t>(qq - q0) * SK_CL_QUAD_BYTES;
        const int nquad = q1 - qq;
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (j < nquad)
            st_shared_v4(dst + j * SK_CL_QUAD_BYTES, v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
      }
      if (!mine) {
        fence_proxy_async_smem();               // the bulk copy reads what was just written
        named_bar_sync(SK_EPI_BAR_ID, SK_EPI_THREADS);
        if (lane == 0 && ((i - 1) & 3) == warp - 2)
          bulk_copy_to_cluster(mapa_shared(recv_base + static_cast<uint32_t>(rank) * chunk_bytes, owner),
                               stage_base + static_cast<uint32_t>(owner) * chunk_bytes, chunk_bytes,
                               mapa_shared(recv_bar, owner));
      }
    }
    tc_fence_before();
    __syncwarp();
    if (lane == 0) mbar_arrive(recv_bar);
    if (warp == 2 && lane == 0) sk_trace(p, 10);
    return;
  }
  // Narrow chunks: the accumulator is read 32 columns at a time in column order, and whatever
  // chunks that completes are sent at once.
  int owner = 0, lq = 0;      // destination CTA and quad inside its chunk of the next quad
  int sent = 0;               // chunks [0, sent) are on their way (or are this CTA's own)
  uint32_t dst = (rank == 0 ? recv_base : stage_base) + row_off;
  for (int c = 0; c < p.bn; c += 32) {
    float v[32];
    if (live) {
      sk_load_acc(t_addr + c, b_off, v);
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = 0.f;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (c + 4 * j < p.bn) {
        st_shared_v4(dst, v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
        dst += SK_CL_QUAD_BYTES;
        if (++lq == per) {
          lq = 0;
          ++owner;
          // the CTA's own chunk goes straight into its receive buffer
          dst = (owner == rank ? recv_base : stage_base) + static_cast<uint32_t>(owner) * chunk_bytes + row_off;
        }
      }
    }
    const int done = (c + 32 >= p.bn) ? S : owner;   // chunks [0, done) are complete
    if (done > sent) {
      fence_proxy_async_smem();               // the bulk copies read what was just written
      named_bar_sync(SK_EPI_BAR_ID, SK_EPI_THREADS);
      if (lane == 0)
        for (int ch = sent + warp - 2; ch < done; ch += 4)
          if (ch != rank)
            bulk_copy_to_cluster(mapa_shared(recv_base + static_cast<uint32_t>(rank) * chunk_bytes, ch),
                                 stage_base + static_cast<uint32_t>(ch) * chunk_bytes, chunk_bytes,
                                 mapa_shared(recv_bar, ch));
      sent = done;
    }
  }
  tc_fence_before();
  __syncwarp();
  if (lane == 0) mbar_arrive(recv_bar);        // this warp's share of the CTA's own chunk is in place
  if (warp == 2 && lane == 0) sk_trace(p, 10);
}

// Step 3; runs on every thread of the CTA once its receive mbarrier has completed.
template <int S>
__device__ __forceinline__ void sk_cluster_reduce_s(const SkParams& p, __half* __restrict__ C, int tile,
                                                    int rank, uint32_t recv_base) {
  using namespace skptx;
  const int per = p.cl_per;
  int tr, tc;
  sk_tile_mn(p.sched, tile, tr, tc);
  const int r0 = tr * p.bm, c0 = tc * p.bn;
  int valid_cols = p.cols - c0;
  if (valid_cols > p.bn) valid_cols = p.bn;
  int nq = ((valid_cols + 3) >> 2) - rank * per;   // quads of this CTA that hold real columns
  if (nq > per) nq = per;
  int rows_valid = p.rows - r0;
  if (rows_valid > p.bm) rows_valid = p.bm;
  const uint32_t chunk_bytes = static_cast<uint32_t>(per) * SK_CL_QUAD_BYTES;
  const int items = per * SK_BM;
  const int gcol0 = c0 + rank * per * 4;
  for (int i = threadIdx.x; i < items; i += blockDim.x) {
    // Consecutive lanes take consecutive rows when C is stored transposed (rows are then
    // contiguous in memory), consecutive quads of one row otherwise.
    int row, lq;
    if (p.transposed) {
      row = i & (SK_BM - 1); lq = i >> 7;
    } else {
      row = sk_div(i, p.cl_per_div); lq = i - row * per;
    }
    if (row >= rows_valid || lq >= nq) continue;
    const uint32_t a = recv_base + static_cast<uint32_t>(lq) * SK_CL_QUAD_BYTES + static_cast<uint32_t>(row) * 16u;
    float4 x[S];
#pragma unroll
    for (int snd = 0; snd < S; ++snd) x[snd] = ld_shared_v4(a + snd * chunk_bytes);
    float4 acc = x[0];
#pragma unroll
    for (int snd = 1; snd < S; ++snd) { acc.x += x[snd].x; acc.y += x[snd].y; acc.z += x[snd].z; acc.w += x[snd].w; }
    sk_store4(C, p, r0 + row, gcol0 + lq * 4, acc);
  }
}

__device__ __forceinline__ void sk_cluster_reduce(const SkParams& p, __half* __restrict__ C, int tile,
                                                  int rank, uint32_t recv_base) {
  switch (p.sched.split) {
    case 2: sk_cluster_reduce_s<2>(p, C, tile, rank, recv_base); break;
    case 4: sk_cluster_reduce_s<4>(p, C, tile, rank, recv_base); break;
    default: sk_cluster_reduce_s<8>(p, C, tile, rank, recv_base); break;
  }
}
