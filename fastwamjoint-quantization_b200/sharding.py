"""Multi-GPU forms of one quantized linear (one process per GPU, ``torch.distributed``).

* Token (M) sharding - the primary form: weights replicated, rank r owns rows ``[r*M/G, (r+1)*M/G)``; rows are
  independent through pre-pass, GEMM and epilogue, so the data path has no collective at all.
* Output-channel (N) split of one wide layer: rank r owns ``W[r*N/G:(r+1)*N/G]`` and computes ``[M, N/G]``;
  the slices are all-gathered (NCCL over NVLink on GPUs, gloo in CPU tests) and laid side by side, optionally in
  token chunks so the gather of one chunk overlaps the GEMM of the next.  The gather moves ``2*M*N*(G-1)/G``
  bytes into every rank and is communication-bound for every shape of interest; it exists because the benchmark
  configuration names it.  Plain NCCL all-gather, no peer-memory kernels.
* The same split with the gather fused into the GEMM (``PeerMatrix`` + ``channel_split_linear_fused``): every rank
  maps the other ranks' output matrices (CUDA IPC) and the GEMM's epilogue stores its block of columns into all of
  them with plain stores over NVLink (``sq_gemm_scatter``); there is no collective and no re-layout afterwards.

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


def channel_split_linear(x: torch.Tensor, linear_slice: Callable[[torch.Tensor], torch.Tensor], *,
                         group=None, chunks: int = 1) -> torch.Tensor:
    """Every rank holds the full ``x`` and a slice of the weight; returns the full ``[..., N]`` output on every
    rank: local GEMM, all-gather of the ``[..., N/G]`` slices, concatenation along the channel axis.

    ``chunks > 1`` cuts the token rows into that many pieces and overlaps communication with compute on CUDA
    devices: the GEMM of piece i + 1 runs on the current stream while the all-gather and the re-layout of piece i
    run on a side stream (NCCL's own kernels; nothing here touches peer memory).  On the CPU (gloo) the pieces
    simply run one after the other, which exercises the same slicing."""
    world = dist.get_world_size(group)
    rows_shape = x.shape[:-1]
    flat_x = x.reshape(-1, x.shape[-1])
    rows = flat_x.shape[0]
    chunks = max(1, min(int(chunks), rows))
    bounds = [row_range(rows, i, chunks) for i in range(chunks)]
    on_gpu = x.is_cuda
    side = torch.cuda.Stream(device=x.device) if on_gpu and chunks > 1 else None
    out = None
    for lo, hi in bounds:
        part = linear_slice(flat_x[lo:hi]).contiguous()
        width = part.shape[-1]
        if out is None:
            out = torch.empty((rows, world * width), dtype=part.dtype, device=part.device)
        gathered = torch.empty((world, hi - lo, width), dtype=part.dtype, device=part.device)

        def gather_and_place(part=part, gathered=gathered, lo=lo, hi=hi, width=width):
            dist.all_gather_into_tensor(gathered.view(world * (hi - lo), width), part, group=group)
            # [G, rows, N/G] -> [rows, G, N/G]: rank r's channels land at columns [r*N/G, (r+1)*N/G)
            out[lo:hi].view(hi - lo, world, width).copy_(gathered.transpose(0, 1))

        if side is None:
            gather_and_place()
        else:
            side.wait_stream(torch.cuda.current_stream(x.device))  # the piece's GEMM has been queued: wait for it
            with torch.cuda.stream(side):
                gather_and_place()
            for tensor in (part, gathered, out):
                tensor.record_stream(side)
    if side is not None:
        torch.cuda.current_stream(x.device).wait_stream(side)
    return out.reshape(*rows_shape, out.shape[-1])


class PeerMatrix:
    """A row-major ``[rows, width]`` matrix of 2-byte elements that exists once per rank and is mapped into every
    other rank of ``group`` through CUDA IPC, so that a kernel of one rank can store into all of them.

    ``pointers[0]`` is this rank's own matrix, the rest are the peers' in rank order (this rank left out).  The
    memory comes straight from ``cudaMalloc`` (an IPC handle names a whole allocation) and is released by
    ``close()``; ``local()`` views this rank's matrix as a torch tensor."""

    def __init__(self, rows: int, width: int, dtype: torch.dtype, *, group=None):
        from cuda.bindings import runtime as rt

        if dtype not in (torch.bfloat16, torch.float16):
            raise ValueError("PeerMatrix holds bf16 or fp16.")
        self._rt, self.rows, self.width, self.dtype, self.group = rt, int(rows), int(width), dtype, group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.device = torch.cuda.current_device()
        nbytes = max(2 * self.rows * self.width, 2)
        err, self._ptr = rt.cudaMalloc(nbytes)
        self._check(err, "cudaMalloc")
        err, handle = rt.cudaIpcGetMemHandle(self._ptr)
        self._check(err, "cudaIpcGetMemHandle")
        handles = [None] * self.world
        dist.all_gather_object(handles, bytes(handle.reserved), group=group)
        self._peers = []
        for rank, raw in enumerate(handles):
            if rank == self.rank:
                continue
            theirs = rt.cudaIpcMemHandle_t()
            theirs.reserved = raw
            err, ptr = rt.cudaIpcOpenMemHandle(theirs, rt.cudaIpcMemLazyEnablePeerAccess)
            self._check(err, f"cudaIpcOpenMemHandle(rank {rank})")
            self._peers.append(int(ptr))
        self.pointers = [int(self._ptr)] + self._peers
        dist.barrier(group=group)

    def _check(self, err, what):
        if int(err) != 0:
            raise RuntimeError(f"{what} failed with CUDA error {int(err)}.")

    def local(self) -> torch.Tensor:
        class _Raw:
            pass

        raw = _Raw()
        raw.__cuda_array_interface__ = {"shape": (self.rows, self.width), "typestr": "<u2", "data": (int(self._ptr), False),
                                        "version": 3, "strides": None}
        self._keep = raw
        return torch.as_tensor(raw, device=f"cuda:{self.device}").view(self.dtype)

    def close(self):
        """Unmap the peers' matrices and free this rank's; every rank must be done with all of them."""
        torch.cuda.synchronize()
        dist.barrier(group=self.group)
        for ptr in self._peers:
            self._rt.cudaIpcCloseMemHandle(ptr)
        self._peers = []
        dist.barrier(group=self.group)
        if self._ptr is not None:
            self._rt.cudaFree(self._ptr)
            self._ptr = None


def channel_split_linear_fused(x: torch.Tensor, packed_slice: torch.Tensor, scales_slice: torch.Tensor, bias_slice,
                               out: PeerMatrix, *, abits: int, signs=None, workspace=None) -> None:
    """Per-token quantized linear of the full ``x`` [rows, K] against this rank's slice of the weight, written into
    this rank's block of columns of ``out`` on EVERY rank by the GEMM's own epilogue (``sq_gemm_scatter``).

    Only queues work on the current stream.  The caller separates calls that reuse ``out`` (a barrier after the
    readers are done) and waits for all ranks (stream synchronize + barrier) before reading ``out.local()``."""
    from . import native

    rows, k = x.shape
    width = packed_slice.shape[0]
    codes, row_scales = native.prepass(x, abits=abits, mode="token", signs=signs, out=workspace)
    native.gemm_scatter(codes, packed_slice, scales_slice, row_scales, bias_slice, out.pointers, out.width,
                        out.rank * width, out_dtype=out.dtype, int4_range=(abits == 4))
