"""Two GPUs, one process each: the channel split with the gather fused into the GEMM's epilogue (sq_gemm_scatter over
CUDA-IPC mapped output matrices) against the whole layer computed on one GPU.  Skipped on boxes with one GPU."""
import os
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]
pytestmark = pytest.mark.gpu


def _worker(rank: int, world: int, port: int, results):
    os.environ.update({"MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port), "NCCL_NVLS_ENABLE": "0"})
    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(ROOT / "oracle"))
    import torch.distributed as dist
    import __graft_entry__ as entry

    entry.load_package()
    import steerquant_oracle as oracle
    from fastwamjoint_quantization_b200 import native, sharding

    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    try:
        m, k, n = 384, 1024, 1024
        case = oracle.prepare_token_linear(m, k, n, abits=4, seed=3)
        x, signs = case["x"].to(device), case["signs"].to(device)
        packed_all = oracle.pack_signed_int4(case["qweight"]).to(device)
        scales_all = case["weight_scales"].to(device)
        whole = native.linear(x, packed_all, scales_all, None, abits=4, mode="token", signs=signs)
        c0, c1 = sharding.channel_range(n, rank, world)
        shared = sharding.PeerMatrix(m, n, torch.bfloat16)
        shared.local().fill_(-1.0)
        torch.cuda.synchronize()
        dist.barrier()
        for _ in range(2):  # the second pass rewrites the same values: reuse of the matrices between barriers
            sharding.channel_split_linear_fused(x, packed_all[c0:c1].contiguous(), scales_all[c0:c1].contiguous(), None,
                                                shared, abits=4, signs=signs)
            torch.cuda.synchronize()
            dist.barrier()
        equal = bool(torch.equal(shared.local(), whole))
        status = native.device_status()
        shared.close()
        results[rank] = (equal, status)
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_fused_channel_split_matches_the_whole_layer_on_two_gpus():
    import torch.multiprocessing as mp

    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(2, 29541, results), nprocs=2, join=True)
    assert dict(results) == {0: (True, 0), 1: (True, 0)}
