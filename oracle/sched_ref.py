"""CPU restatement of the reference's Stream-K work decomposition.  Test infrastructure."""
from __future__ import annotations


def cdiv(a: int, b: int) -> int:
    return -(-a // b)


def reference_schedule(M: int, N: int, K: int, BM: int, BN: int, BK: int, P: int) -> dict:
    """The host integers of streamk_fp16.py:83-113 (same in every Stream-K script and in
    triton_impl.py:205-219), with the variable names of the reference."""
    num_block_m = cdiv(M, BM)
    num_block_n = cdiv(N, BN)
    iters_per_tile = cdiv(K, BK)
    total_tiles = num_block_m * num_block_n
    streamk_tiles = total_tiles % P
    if total_tiles - streamk_tiles > P:      # "two-tile SK + DP"
        streamk_tiles += P
    blocking_tiles = total_tiles - streamk_tiles
    streamk_iters = streamk_tiles * iters_per_tile
    return dict(num_block_m=num_block_m, num_block_n=num_block_n, iters_per_tile=iters_per_tile,
                total_tiles=total_tiles, streamk_tiles=streamk_tiles, blocking_tiles=blocking_tiles,
                streamk_iters=streamk_iters, streamk_full_tiles=streamk_iters // P,
                streamk_partial_tiles=streamk_iters % P)


def cta_segments(pid: int, *, sk_tiles: int, total_tiles: int, iters_per_tile: int, grid: int,
                 full: int, partial: int, dp_first: bool = False):
    """Segments (tile, k0, k1) CTA `pid` executes, in order.

    Stream-K part: the interval walk of streamk_fp16.py:176-193
    (start = pid*full + min(pid, partial); segment ends at the tile boundary or at the
    interval end).  Data-parallel part: tile = pid + sk_tiles + w*grid
    (streamk_fp16.py:274-275), for as many waves as have a tile (the reference always
    runs max(blocking // P, 1) waves, which over-runs when there are none)."""
    sk = []
    start = pid * full + min(pid, partial)
    last = (pid + 1) * full + min(pid + 1, partial)
    while start < last:
        end = min(start + (iters_per_tile - start % iters_per_tile), last)
        sk.append((start // iters_per_tile, start % iters_per_tile,
                   start % iters_per_tile + (end - start)))
        start = end
    dp = []
    w = 0
    while sk_tiles + pid + w * grid < total_tiles:
        dp.append((sk_tiles + pid + w * grid, 0, iters_per_tile))
        w += 1
    return dp + sk if dp_first else sk + dp


def cluster_segments(pid: int, *, iters_per_tile: int, cluster: int):
    """Split-K inside a thread-block cluster (no counterpart in the reference): CTA `pid`
    is rank r = pid % cluster of tile pid // cluster and walks K iterations
    [r*I // cluster, (r+1)*I // cluster) of it; nothing if that range is empty."""
    tile, r = divmod(pid, cluster)
    k0, k1 = r * iters_per_tile // cluster, (r + 1) * iters_per_tile // cluster
    return [(tile, k0, k1)] if k1 > k0 else []


def coverage(sched: dict) -> dict:
    """(tile, k) -> number of times covered, over all CTAs of a schedule described by the
    library's sk_schedule_info fields."""
    cover: dict = {}
    for pid in range(sched["grid"]):
        if sched.get("cluster", 0) > 0:
            for tile, k0, k1 in cluster_segments(pid, iters_per_tile=sched["iters_per_tile"],
                                                 cluster=sched["cluster"]):
                for k in range(k0, k1):
                    cover[(tile, k)] = cover.get((tile, k), 0) + 1
            continue
        for tile, k0, k1 in cta_segments(pid, sk_tiles=sched["sk_tiles"],
                                         total_tiles=sched["total_tiles"],
                                         iters_per_tile=sched["iters_per_tile"],
                                         grid=sched["grid"], full=sched["sk_iters_per_cta"],
                                         partial=sched["sk_iters_rem"],
                                         dp_first=bool(sched["dp_first"])):
            for k in range(k0, k1):
                cover[(tile, k)] = cover.get((tile, k), 0) + 1
    return cover


def tile_coords(tile: int, tiles_m: int, tiles_n: int, group_m: int = 1):
    """Row-major order is the reference's (streamk_fp16.py:192-193).  group_m > 1 is a
    grouped order in the spirit of its unused swizzle_tile (triton_impl.py:14-28): bands
    of group_m tile rows, column-major inside a band (a bijection for ragged bands too)."""
    if group_m <= 1:
        return tile // tiles_n, tile % tiles_n
    width = group_m * tiles_n
    g = tile // width
    first_m = g * group_m
    gsize = min(tiles_m - first_m, group_m)
    return first_m + (tile % width) % gsize, (tile % width) // gsize
