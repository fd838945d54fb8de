"""The multi-GPU host logic on CPU: two gloo ranks, a stand-in for the rank-local quantized linear."""
import importlib
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, results):
    import sys
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import __graft_entry__ as entry
    entry.load_package()
    sharding = importlib.import_module("fastwamjoint_quantization_b200.sharding")
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        gen = torch.Generator().manual_seed(0)
        # small integers: every product and sum is exact, whatever the row count of a matmul call
        x = torch.randint(-4, 5, (10, 16), generator=gen).float()
        w = torch.randint(-4, 5, (24, 16), generator=gen).float()
        full = x @ w.t()
        # tokens sharded, weights replicated: no communication, ranks' rows tile the full result
        lo, hi = sharding.row_range(10, rank, world)
        local = x[lo:hi] @ w.t()  # rank-local rows in, rank-local rows out: nothing to call
        ok_rows = torch.equal(local, full[lo:hi])
        # channels split, all-gather
        c0, c1 = sharding.channel_range(24, rank, world, multiple=4)
        gathered = sharding.channel_split_linear(x, lambda t: t @ w[c0:c1].t())
        ok_cols = torch.equal(gathered, full)
        for chunks in (2, 3, 64):  # token chunks (the form that overlaps gather and GEMM on GPUs), ragged and over-split
            piecewise = sharding.channel_split_linear(x.reshape(2, 5, 16), lambda t: t @ w[c0:c1].t(), chunks=chunks)
            ok_cols = ok_cols and torch.equal(piecewise, full.reshape(2, 5, 24))
        results[rank] = (ok_rows, ok_cols, (lo, hi), (c0, c1))
    finally:
        dist.destroy_process_group()


def test_two_rank_sharding_on_gloo():
    world, port = 2, _free_port()
    manager = mp.get_context("spawn").Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
    assert results[0][:2] == (True, True) and results[1][:2] == (True, True)
    assert results[0][2] == (0, 5) and results[1][2] == (5, 10)
    assert results[0][3] == (0, 12) and results[1][3] == (12, 24)


def test_ranges(pkg):
    sharding = importlib.import_module("fastwamjoint_quantization_b200.sharding")
    spans = [sharding.row_range(1592, r, 8) for r in range(8)]
    assert spans[0] == (0, 199) and spans[-1] == (1393, 1592)
    assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
    assert [sharding.row_range(16, r, 8)[1] - sharding.row_range(16, r, 8)[0] for r in range(8)] == [2] * 8
    assert sharding.row_range(3, 2, 4) == (2, 3) and sharding.row_range(3, 3, 4) == (3, 3)
    assert sharding.channel_range(12288, 7, 8) == (10752, 12288)
    with pytest.raises(ValueError):
        sharding.channel_range(100, 0, 8)
    with pytest.raises(ValueError):
        sharding.row_range(10, 4, 4)
