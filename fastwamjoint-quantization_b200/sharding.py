"""Multi-GPU forms of one quantized linear (one process per GPU, ``torch.distributed``).

* Token (M) sharding - the primary form: weights replicated, rank r owns rows ``[r*M/G, (r+1)*M/G)``; rows are
  independent through pre-pass, GEMM and epilogue, so the data path has no collective at all.
* Output-channel (N) split of one wide layer: rank r owns ``W[r*N/G:(r+1)*N/G]`` and computes ``[M, N/G]``;
  the slices are all-gathered (NCCL over NVLink on GPUs, gloo in CPU tests) and laid side by side.  The
  gather moves ``2*M*N*(G-1)/G`` bytes per rank and is communication-bound for every shape of interest; it
  exists because the benchmark configuration names it.  Plain NCCL all-gather, no peer-memory kernels.

The host-side logic (row ranges, slice ownership, gather + re-layout) is device independent and is tested
with world-size-2 gloo process groups on CPU with a stand-in for the local linear.
"""
from __future__ import annotations

from typing import Callable

import torch
import torch.distributed as dist


def row_range(rows: int, rank: int, world: int) -> tuple[int, int]:
    """Contiguous, balanced split of ``rows``: the first ``rows % world`` ranks get one extra row."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError("rank must lie in [0, world).")
    base, extra = divmod(int(rows), world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def channel_range(channels: int, rank: int, world: int, multiple: int = 8) -> tuple[int, int]:
    """Equal split of output channels; each slice must keep the kernels' N % 8 alignment."""
    if channels % world or (channels // world) % multiple:
        raise ValueError(f"{channels} output channels do not split into {world} slices of a multiple of {multiple}.")
    width = channels // world
    return rank * width, (rank + 1) * width


def token_sharded_linear(x_local: torch.Tensor, linear: Callable[[torch.Tensor], torch.Tensor]) -> torch.Tensor:
    """Rank-local rows in, rank-local rows out: no communication."""
    return linear(x_local)


def channel_split_linear(x: torch.Tensor, linear_slice: Callable[[torch.Tensor], torch.Tensor], *,
                         group=None) -> torch.Tensor:
    """Every rank holds the full ``x`` and a slice of the weight; returns the full ``[..., N]`` output on every
    rank: local GEMM, all-gather of the ``[..., N/G]`` slices, concatenation along the channel axis."""
    part = linear_slice(x).contiguous()
    world = dist.get_world_size(group)
    flat = part.reshape(-1, part.shape[-1])
    gathered = torch.empty((world * flat.shape[0], flat.shape[1]), dtype=part.dtype, device=part.device)
    dist.all_gather_into_tensor(gathered, flat, group=group)  # rank-major concatenation of the slices
    # [G, rows, N/G] -> [rows, G, N/G] -> [..., N]
    wide = gathered.reshape(world, flat.shape[0], flat.shape[1]).transpose(0, 1)
    return wide.reshape(*part.shape[:-1], world * part.shape[-1])
