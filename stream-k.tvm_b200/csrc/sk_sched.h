// Stream-K work decomposition shared by host and device code.
//
// Follows the host arithmetic of the reference (streamk_fp16.py:83-113) and the
// per-CTA interval walk of its kernels (streamk_fp16.py:176-193, 274-277), with
// the defects removed: no data-parallel pass is run when there are no
// data-parallel tiles, and a ragged last data-parallel wave is allowed.
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define SK_HD __host__ __device__ __forceinline__
#else
#define SK_HD inline
#endif

// Division by a number known on the host, as multiply-high and shift (valid for
// 0 <= n < 2^31): the device walks the schedule in a single thread, where a plain integer
// division is some thirty dependent instructions.
struct SkDiv {
  uint32_t mul;   // 0: the divisor is 1
  uint32_t shr;
};

SK_HD SkDiv sk_div_make(int d) {
  SkDiv v;
  v.mul = 0; v.shr = 0;
  if (d <= 1) return v;
  int l = 0;
  while ((1u << l) < static_cast<uint32_t>(d)) ++l;   // ceil(log2 d)
  const int p = 31 + l;
  v.mul = static_cast<uint32_t>(((1ull << p) + static_cast<uint32_t>(d) - 1) / static_cast<uint32_t>(d));
  v.shr = static_cast<uint32_t>(p - 32);
  return v;
}

SK_HD int sk_div(int n, const SkDiv& d) {
  if (d.mul == 0) return n;
#if defined(__CUDA_ARCH__)
  return static_cast<int>(__umulhi(static_cast<uint32_t>(n), d.mul) >> d.shr);
#else
  return static_cast<int>(static_cast<uint32_t>((static_cast<uint64_t>(static_cast<uint32_t>(n)) * d.mul) >> 32) >> d.shr);
#endif
}

struct SkSched {
  int tiles_m, tiles_n, total_tiles, iters_per_tile;
  int sk_tiles;   // tiles [0, sk_tiles) are Stream-K'd
  int grid;       // persistent CTAs
  int sk_f;       // iterations per CTA (floor)      "streamk_full_tiles"
  int sk_r;       // CTAs that get one more          "streamk_partial_tiles"
  int dp_first;   // 1: data-parallel waves before the Stream-K part
  int group_m;    // rasterisation group height in tiles (1 = row-major)
  int split;      // > 0: every tile is split over the `split` CTAs of one thread-block cluster
                  //      (grid = total_tiles * split), CTA r of the cluster walking K iterations
                  //      [r*I/split, (r+1)*I/split) of its tile; 0: the Stream-K interval rule
  int wide_base;  // >= 0: see sk_tile_mn; -1: tiles are rasterised directly
  // derived by sk_sched_finish()
  int split_log2; // split is a power of two
  SkDiv d_ipt;    // / iters_per_tile
  SkDiv d_tn;     // / tiles_n
  SkDiv d_width;  // / (group_m * tiles_n)
  SkDiv d_gm;     // / group_m
  SkDiv d_glast;  // / height of the ragged last band
  SkDiv d_f1;     // / (sk_f + 1)
  SkDiv d_f;      // / sk_f
};

// Fill the derived fields once the others are set.
SK_HD void sk_sched_finish(SkSched& s) {
  s.split_log2 = 0;
  while ((1 << s.split_log2) < s.split) ++s.split_log2;
  s.d_ipt = sk_div_make(s.iters_per_tile);
  s.d_tn = sk_div_make(s.tiles_n);
  const int gm = s.group_m > 1 ? s.group_m : 1;
  s.d_width = sk_div_make(gm * s.tiles_n);
  s.d_gm = sk_div_make(gm);
  const int last = s.tiles_m % gm;
  s.d_glast = sk_div_make(last ? last : gm);
  s.d_f1 = sk_div_make(s.sk_f + 1);
  s.d_f = sk_div_make(s.sk_f > 0 ? s.sk_f : 1);
}

struct SkSeg {
  int tile;
  int k0, k1;     // iteration range inside the tile, [k0, k1) of iters_per_tile
};

struct SkCursor {
  int stage;      // 0 first phase, 1 second phase, 2 done
  int it, it_end; // Stream-K iteration cursor
  int dp_w;       // next data-parallel wave
};

// First iteration of CTA p: p*f + min(p, r)   (streamk_fp16.py:176-181)
SK_HD int sk_cta_begin(const SkSched& s, int p) {
  if (s.split > 0) {
    const int t = p >> s.split_log2, r = p & (s.split - 1);
    // r < split <= 16 and iters_per_tile < 2^27: the product fits 32 bits
    return t * s.iters_per_tile + ((r * s.iters_per_tile) >> s.split_log2);
  }
  return p * s.sk_f + (p < s.sk_r ? p : s.sk_r);
}

// Inverse of sk_cta_begin: which CTA executes Stream-K iteration i.
SK_HD int sk_cta_of(const SkSched& s, int i) {
  if (s.split > 0) {
    const int t = sk_div(i, s.d_ipt), k = i - t * s.iters_per_tile;
    return t * s.split + sk_div((k + 1) * s.split - 1, s.d_ipt);
  }
  const int big = s.sk_r * (s.sk_f + 1);
  if (i < big) return sk_div(i, s.d_f1);
  return s.sk_r + sk_div(i - big, s.d_f);   // sk_f > 0 here, else i < big always
}

// Tile id -> tile coordinates.  group_m == 1 is the reference's row-major order
// (streamk_fp16.py:192-193); group_m > 1 walks column-major inside bands of
// group_m tile rows so that a wave of CTAs shares A and B panels in L2.
SK_HD void sk_raster_mn(const SkSched& s, int tile, int& tm, int& tn) {
  if (s.group_m <= 1) {
    tm = sk_div(tile, s.d_tn);
    tn = tile - tm * s.tiles_n;
    return;
  }
  const int g = sk_div(tile, s.d_width);
  const int first_m = g * s.group_m;
  const int rem = s.tiles_m - first_m;
  const bool full = rem >= s.group_m;
  const int gsize = full ? s.group_m : rem;
  const int in_g = tile - g * (s.group_m * s.tiles_n);
  tn = sk_div(in_g, full ? s.d_gm : s.d_glast);
  tm = first_m + (in_g - tn * gsize);
}

// Tile id of the schedule -> tile coordinates.  With wide_base >= 0 (CTA-pair kernel, see
// sk_gemm_f16_2cta.cu) the rasterised grid is one of UNITS two tiles wide, its first wide_base
// units are walked whole by another part of the kernel, and the schedule's tiles are the halves
// of the remaining units: tile t = half t & 1 of unit wide_base + t / 2.
SK_HD void sk_tile_mn(const SkSched& s, int tile, int& tm, int& tn) {
  if (s.wide_base < 0) {
    sk_raster_mn(s, tile, tm, tn);
    return;
  }
  sk_raster_mn(s, s.wide_base + (tile >> 1), tm, tn);
  tn = 2 * tn + (tile & 1);
}

SK_HD void sk_cursor_init(const SkSched& s, int pid, SkCursor& c) {
  c.stage = 0;
  c.it = sk_cta_begin(s, pid);
  c.it_end = sk_cta_begin(s, pid + 1);
  c.dp_w = 0;
}

// Next work segment of CTA pid, or false when it has none left.
SK_HD bool sk_next(const SkSched& s, int pid, SkCursor& c, SkSeg& seg) {
  while (c.stage < 2) {
    const bool sk_phase = (c.stage == 0) != (s.dp_first != 0);
    if (sk_phase) {
      if (c.it < c.it_end) {
        const int I = s.iters_per_tile;
        const int tile = sk_div(c.it, s.d_ipt);
        const int k0 = c.it - tile * I;
        int k1 = k0 + (c.it_end - c.it);
        if (k1 > I) k1 = I;
        seg.tile = tile; seg.k0 = k0; seg.k1 = k1;
        c.it += k1 - k0;
        return true;
      }
    } else {
      const int tile = s.sk_tiles + pid + c.dp_w * s.grid;
      if (tile < s.total_tiles) {
        seg.tile = tile; seg.k0 = 0; seg.k1 = s.iters_per_tile;
        c.dp_w++;
        return true;
      }
    }
    c.stage++;
  }
  return false;
}

// CTAs that contribute to Stream-K tile `tile`: [first, last].
SK_HD void sk_tile_ctas(const SkSched& s, int tile, int& first, int& last) {
  const int I = s.iters_per_tile;
  first = sk_cta_of(s, tile * I);
  last = sk_cta_of(s, tile * I + I - 1);
}
