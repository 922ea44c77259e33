// Epilogue shared by the tensor-core kernels: TMEM accumulator -> fp16 C, or the
// cross-CTA fixup of a partial tile.
//
// Two fixups, both on fp32 partial sums (the reference adds fp16 halves straight
// into a pre-zeroed C with T.atomic_addx2, streamk_fp16.py:248-255):
//   atomic        every contributor red.global.add's its partial into the tile's
//                 zero-kept slot; the last one to arrive (a counter tells) folds the
//                 slot into C and zeroes it again.
//   block_reduce  contributors other than the tile owner publish their partial and
//                 a flag; the owner (the CTA that computed the tile's first K
//                 iteration, which it reaches last) waits with a time limit, adds the
//                 partials in ascending CTA order and stores C.  The order is fixed,
//                 so the result is bitwise reproducible.
// Slot layout (private): float4 index = (column / 4) * 128 + row, so a warp's 32
// rows write 512 contiguous bytes per instruction.
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

// 32 fp32 values of one row -> fp16 -> C[row, col0 .. col0+31]
__device__ __forceinline__ void sk_store_c_row(__half* __restrict__ C, const SkParams& p, int grow,
                                            int gcol0, const float (&v)[32]) {
  __half* dst = C + static_cast<size_t>(grow) * p.ldc + gcol0;
  if (p.c_vec_ok && gcol0 + 32 <= p.N) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      __half2 h0 = __floats2half2_rn(v[8 * j + 0], v[8 * j + 1]);
      __half2 h1 = __floats2half2_rn(v[8 * j + 2], v[8 * j + 3]);
      __half2 h2 = __floats2half2_rn(v[8 * j + 4], v[8 * j + 5]);
      __half2 h3 = __floats2half2_rn(v[8 * j + 6], v[8 * j + 7]);
      uint4 u;
      u.x = *reinterpret_cast<uint32_t*>(&h0);
      u.y = *reinterpret_cast<uint32_t*>(&h1);
      u.z = *reinterpret_cast<uint32_t*>(&h2);
      u.w = *reinterpret_cast<uint32_t*>(&h3);
      *reinterpret_cast<uint4*>(dst + 8 * j) = u;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (gcol0 + j < p.N) dst[j] = __float2half_rn(v[j]);
  }
}

// Runs on the four epilogue warps (any four consecutive warps; `warp & 3` picks the
// TMEM lane quadrant a warp may read).  tmem_full_bar / tmem_empty_bar are the
// shared-memory addresses of two consecutive mbarriers each (one per accumulator).
template <int BN>
__device__ __forceinline__ void sk_epilogue_loop(const SkParams& p, __half* __restrict__ C, int pid,
                                                 int warp, int lane, uint32_t tmem_base,
                                                 uint32_t tmem_full_bar, uint32_t tmem_empty_bar,
                                                 volatile uint32_t* bcast,
                                                 volatile uint32_t* abort_flag) {
  using namespace skptx;
  constexpr int BM = SK_BM;
  constexpr int EPI_THREADS = SK_EPI_THREADS;
  constexpr int EPI_BAR_ID = SK_EPI_BAR_ID;
  constexpr size_t SLOT_FLOATS = SK_SLOT_BYTES / sizeof(float);
  const SkSched& s = p.sched;
  const int q = warp & 3;            // TMEM lane quadrant this warp may read
  const int row = q * 32 + lane;     // row inside the tile
  const int etid = ((warp - 2) & 3) * 32 + lane;
  SkCursor cur;
  sk_cursor_init(s, pid, cur);
  SkSeg seg;
  uint32_t nseg = 0;
  bool dead = false;
  while (sk_next(s, pid, cur, seg)) {
    const uint32_t buf = nseg & 1u;
    const uint32_t acc_ph = (nseg >> 1) & 1u;
    ++nseg;
    int tm, tn;
    sk_tile_mn(s, seg.tile, tm, tn);
    const int m0 = tm * BM, n0 = tn * BN;
    const int grow = m0 + row;
    const bool row_ok = grow < p.M;
    const bool warp_ok = (m0 + q * 32) < p.M;  // warp-uniform
    int nchunks = (p.N - n0 + 31) / 32;
    if (nchunks > BN / 32) nchunks = BN / 32;
    const bool whole = (seg.k0 == 0 && seg.k1 == s.iters_per_tile);
    int first = 0, last = 0;
    if (!whole) sk_tile_ctas(s, seg.tile, first, last);
    const bool owner = !whole && p.fixup == SK_FIXUP_BLOCK_REDUCE && seg.k0 == 0;

    // The owner waits for its peers' partials before it touches TMEM so that the
    // registers it loads can be finished column chunk by column chunk.
    bool peers_ok = true;
    if (owner) {
      if (etid == 0) {
        uint32_t ok = 1u;
        for (int peer = first + 1; peer <= last; ++peer) {
          if (!sk_wait_flag(p.ws.flags + peer, p.timeout_ns)) {
            sk_report(p.ws.status, SK_ERR_FIXUP_TIMEOUT, seg.tile, peer);
            ok = 0u;
            break;
          }
        }
        *bcast = ok;
      }
      named_bar_sync(EPI_BAR_ID, EPI_THREADS);
      peers_ok = *bcast != 0u;
    }

    // A wait that ran out must not leave the warps disagreeing: every epilogue
    // thread keeps walking the segment list (and meeting the named barriers) but
    // stops touching tensor memory.
    if (!dead) {
      const bool got = sk_wait_bar(tmem_full_bar + 8u * buf, acc_ph, abort_flag, p, 24 + buf, 2);
      if (!__all_sync(0xffffffffu, got)) dead = true;
    }
    tc_fence_after();
    if (nseg == 1 && etid == 0) sk_trace(p, 5);
    const uint32_t t_addr = tmem_base + buf * BN + (static_cast<uint32_t>(q * 32) << 16);

    float* acc_slot = p.ws.acc_slots + static_cast<size_t>(first) * SLOT_FLOATS;
    float* my_part = p.ws.part_slots + static_cast<size_t>(pid) * SLOT_FLOATS;

    if (warp_ok && !dead) {
      for (int c = 0; c < nchunks; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(t_addr + c * 32, r);
        tmem_ld_wait();
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
        if (!row_ok) continue;
        if (whole) {
          sk_store_c_row(C, p, grow, n0 + c * 32, v);
        } else if (p.fixup == SK_FIXUP_ATOMIC) {
#pragma unroll
          for (int j = 0; j < 8; ++j)
            red_add_v4(acc_slot + (static_cast<size_t>(c * 8 + j) * BM + row) * 4, v[4 * j],
                       v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
        } else if (!owner) {
#pragma unroll
          for (int j = 0; j < 8; ++j)
            __stcg(reinterpret_cast<float4*>(my_part + (static_cast<size_t>(c * 8 + j) * BM + row) * 4),
                   make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]));
        } else if (peers_ok) {
          for (int peer = first + 1; peer <= last; ++peer) {
            const float* part = p.ws.part_slots + static_cast<size_t>(peer) * SLOT_FLOATS;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float4 x = __ldcg(reinterpret_cast<const float4*>(
                  part + (static_cast<size_t>(c * 8 + j) * BM + row) * 4));
              v[4 * j] += x.x; v[4 * j + 1] += x.y; v[4 * j + 2] += x.z; v[4 * j + 3] += x.w;
            }
          }
          sk_store_c_row(C, p, grow, n0 + c * 32, v);
        }
      }
    }
    // hand the accumulator back to the MMA warp
    tc_fence_before();
    __syncwarp();
    if (lane == 0) mbar_arrive(tmem_empty_bar + 8u * buf);

    if (whole) continue;
    if (p.fixup == SK_FIXUP_ATOMIC) {
      __threadfence();
      named_bar_sync(EPI_BAR_ID, EPI_THREADS);
      if (etid == 0) {
        const uint32_t old = atom_add_acqrel_u32(p.ws.counters + first, 1u);
        *bcast = (old == static_cast<uint32_t>(last - first)) ? 1u : 0u;
      }
      named_bar_sync(EPI_BAR_ID, EPI_THREADS);
      if (*bcast != 0u) {
        // last contributor: fold the slot into C and leave the slot zeroed
        __threadfence();
        if (row_ok) {
          for (int c = 0; c < nchunks; ++c) {
            float v[32];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              float4* q4 = reinterpret_cast<float4*>(
                  acc_slot + (static_cast<size_t>(c * 8 + j) * BM + row) * 4);
              const float4 x = __ldcg(q4);
              __stcg(q4, make_float4(0.f, 0.f, 0.f, 0.f));
              v[4 * j] = x.x; v[4 * j + 1] = x.y; v[4 * j + 2] = x.z; v[4 * j + 3] = x.w;
            }
            sk_store_c_row(C, p, grow, n0 + c * 32, v);
          }
        }
        if (etid == 0) p.ws.counters[first] = 0u;
      }
      named_bar_sync(EPI_BAR_ID, EPI_THREADS);  // bcast is reused by the next segment
    } else if (!owner) {
      __threadfence();
      named_bar_sync(EPI_BAR_ID, EPI_THREADS);
      if (etid == 0 && pid != p.drop_flag_cta) st_release_u32(p.ws.flags + pid, 1u);
    } else {
      named_bar_sync(EPI_BAR_ID, EPI_THREADS);  // every thread has read the partials
      if (etid == 0 && peers_ok)
        for (int peer = first + 1; peer <= last; ++peer) p.ws.flags[peer] = 0u;
    }
  }
  if (etid == 0) sk_trace(p, 6);
}
