"""Host-side logic of the sharded configuration (N split across ranks), run as two gloo
ranks on the CPU: slab bounds, per-slab schedule, and that the slabs' oracle results tile
the full result.  No GPU and no library compute call is involved."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, out_dir: str):
    sys.path.insert(0, ROOT)
    import oracle
    import streamk_b200 as sk
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        M, N, K = 64, 512, 256                      # scaled-down configuration 5
        g = torch.Generator().manual_seed(5000)
        A = torch.randn(M, K, generator=g).half()
        slabs = [oracle.inputs.slab_case(s, N // 8, K) for s in range(8)]   # same B on every rank
        per = 8 // world
        mine = torch.cat(slabs[rank * per:(rank + 1) * per], 0)
        assert mine.shape == (N // world, K)
        C_slab = oracle.gemm_ref(A, mine, "nt")
        # every rank plans its own slab with the library's host scheduler
        info = sk.schedule_info(M, N // world, K, schedule="hybrid", num_sms=148)
        assert info["total_tiles"] * info["iters_per_tile"] > 0
        # gather the column blocks the way bench.py does (all_gather then permute)
        parts = [torch.empty_like(C_slab) for _ in range(world)]
        dist.all_gather(parts, C_slab)
        C_full = torch.cat(parts, 1)
        ref = oracle.gemm_ref(A, torch.cat(slabs, 0), "nt")
        assert torch.equal(C_full, ref)
        # the fused gather's host logic: equal aligned column blocks, each rank writing to its
        # peers in an order of its own (no two ranks address the same destination at once)
        col0, width = sk.column_block(rank, world, N)
        assert (col0, width) == (rank * N // world, N // world)
        assert torch.equal(C_full[:, col0:col0 + width], C_slab)
        orders = [None] * world
        dist.all_gather_object(orders, sk.peer_order(rank, world))
        for step in range(world - 1):
            assert sorted(o[step] for o in orders) == list(range(world))
        assert all(r not in orders[r] for r in range(world))
        # no GPU here: the shared result matrices cannot be made, and every rank says so (none
        # is left waiting in a collective call for a rank that gave up)
        if not torch.cuda.is_available():
            with pytest.raises(Exception):
                sk.GatheredResult(M, N, device="cuda:0")
        # max-over-ranks timing reduction used by the benchmark
        t = torch.tensor([float(rank + 1)], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        assert t.item() == world
        open(os.path.join(out_dir, f"ok{rank}"), "w").write("ok")
    finally:
        dist.destroy_process_group()


def test_two_rank_sharding_on_cpu(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all(os.path.exists(tmp_path / f"ok{r}") for r in range(world))


def test_bench_operand_slabs_are_world_size_independent():
    sys.path.insert(0, ROOT)
    import bench
    assert bench.N5 % 8 == 0 and bench.BASE_SLAB * 8 == bench.N5
    for world in (1, 2, 4, 8):
        assert (bench.N5 // world) % 256 == 0       # whole 256-column tiles per GPU


def test_gather_layout_rules():
    sys.path.insert(0, ROOT)
    import streamk_b200 as sk
    assert sk.column_block(3, 8, 28672) == (3 * 3584, 3584)
    assert sk.peer_order(0, 1) == [] and sk.peer_order(6, 8) == [7, 0, 1, 2, 3, 4, 5]
    with pytest.raises(ValueError):
        sk.column_block(0, 3, 28672)        # does not divide
    with pytest.raises(ValueError):
        sk.column_block(0, 2, 24)           # blocks of 12 columns: not 16-byte aligned
    with pytest.raises(ValueError):
        sk.column_block(2, 2, 1024)
