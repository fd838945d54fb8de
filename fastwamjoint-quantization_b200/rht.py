"""Seeded signs and block Hadamard rotation used to prepare weights (and as the reference form of the
activation rotation).  Semantics of the reference's ``rht.py``: ``rht_signs`` is bit-identical
(``rht.py:81-96``); ``block_hadamard`` is ``_normalized_block_hadamard`` (``rht.py:99-112``) with the block
length given explicitly instead of derived from the width."""
from __future__ import annotations

import hashlib
import math

import torch

RHT_BLOCK = 128


def rht_block_size(width: int) -> int:
    """Largest power of two dividing ``width`` (``rht.py:69-78``)."""
    width = int(width)
    if width <= 0:
        raise ValueError(f"RHT input width must be positive, got {width}.")
    block = width & -width
    if block < 2:
        raise ValueError(f"RHT requires an even input width, got {width}.")
    return block


def rht_signs(in_features: int, *, seed: int, module_name: str, device=None) -> torch.Tensor:
    """Reproducible +-1 vector: sha256 of ``"{seed}:{module_name}"`` seeds a CPU generator."""
    rht_block_size(in_features)
    digest = hashlib.sha256(f"{int(seed)}:{module_name}".encode()).digest()
    generator = torch.Generator(device="cpu").manual_seed(int.from_bytes(digest[:8], "little") % (2**63 - 1))
    bits = torch.randint(0, 2, (int(in_features),), generator=generator, dtype=torch.int8)
    signs = (bits * 2 - 1).float()
    return signs if device is None else signs.to(device=device)


def block_hadamard(values: torch.Tensor, block: int = RHT_BLOCK) -> torch.Tensor:
    """Normalised Sylvester-order Hadamard transform of every ``block``-long piece of the last axis,
    butterfly strides 1, 2, 4, ... then one multiply by ``1/sqrt(block)``."""
    width = int(values.shape[-1])
    if block <= 0 or block & (block - 1) or width % block:
        raise ValueError("block must be a power of two dividing the width.")
    work = values.float().reshape(-1, width // block, block).clone()
    stride = 1
    while stride < block:
        view = work.reshape(-1, width // block, block // (2 * stride), 2, stride)
        lo, hi = view[..., 0, :].clone(), view[..., 1, :].clone()
        view[..., 0, :] = lo + hi
        view[..., 1, :] = lo - hi
        stride *= 2
    return work.reshape(values.shape) * (1.0 / math.sqrt(block))


def randomized_block_hadamard_transform(values: torch.Tensor, signs: torch.Tensor, block: int | None = None):
    """``block_hadamard(values * signs)``; ``block=None`` uses the reference's rule (largest power of two
    dividing the width, ``rht.py:115-145``)."""
    if values.ndim == 0:
        raise ValueError("RHT input must have a final hidden dimension.")
    width = int(values.shape[-1])
    if tuple(signs.shape) != (width,):
        raise ValueError(f"RHT signs must have shape [{width}], got {tuple(signs.shape)}.")
    block = rht_block_size(width) if block is None else block
    return block_hadamard(values * signs.to(device=values.device, dtype=values.dtype), block)


def composite_order(width: int) -> int | None:
    """Order of the sign matrix the reference's "rht" rotation uses for this width (``rht.py:31-34``):
    12 at 3072, 28 at 14336, none for powers of two (plain FWHT)."""
    return {3072: 12, 14336: 28}.get(int(width))


def composite_hadamard(values: torch.Tensor, matrix: torch.Tensor) -> torch.Tensor:
    """``rht.py:27-39`` with the sign matrix as an argument: view the last axis as ``[order, P]`` (P a power of
    two), normalised FWHT of every row, the matrix across the rows, one division by ``sqrt(order)``.  The
    order-12 / order-28 matrices belong to the checkpoint's tooling and are passed in by the caller."""
    order = int(matrix.shape[0])
    width = int(values.shape[-1])
    if matrix.ndim != 2 or matrix.shape[1] != order or width % order:
        raise ValueError("matrix must be square and its order must divide the width.")
    part = width // order
    if part & (part - 1):
        raise ValueError("width / order must be a power of two.")
    transformed = block_hadamard(values.float().reshape(-1, order, part), part)
    mixed = matrix.to(device=values.device, dtype=torch.float32) @ transformed
    return mixed.reshape(values.shape) / torch.full((), math.sqrt(order), device=values.device)


def randomized_composite_hadamard_transform(values: torch.Tensor, signs: torch.Tensor, matrix: torch.Tensor):
    """``composite_hadamard(values * signs)`` (``rht.py:45-46, 56-59``)."""
    if values.ndim == 0 or tuple(signs.shape) != (values.shape[-1],):
        raise ValueError("Official RHT requires one sign per input channel.")
    return composite_hadamard(values * signs.to(device=values.device, dtype=values.dtype), matrix)


def rotate_weight_(weight: torch.Tensor, signs: torch.Tensor, block: int = RHT_BLOCK, rows_per_step: int = 128):
    """Rotate a Linear weight in place along its input axis: fp32 rotate, round back to the weight's dtype
    (``rht_install.py:39-41``), in row chunks so no second fp32 copy of a wide matrix exists."""
    for start in range(0, weight.shape[0], rows_per_step):
        rows = weight[start:start + rows_per_step]
        rows.copy_(randomized_block_hadamard_transform(rows.float(), signs, block).to(rows.dtype))
    return weight
