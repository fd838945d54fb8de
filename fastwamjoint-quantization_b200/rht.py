"""Seeded signs and block Hadamard rotation used to prepare weights (and as the reference form of the
activation rotation).  Semantics of the reference's ``rht.py``: ``rht_signs`` is bit-identical
(``rht.py:81-96``); ``block_hadamard`` is ``_normalized_block_hadamard`` (``rht.py:99-112``) with the block
length given explicitly instead of derived from the width."""
from __future__ import annotations

import hashlib
import math
from functools import lru_cache

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


# Rows of the order-12 and order-28 Hadamard matrices the reference's "rht" rotation uses, one bit mask per row
# (bit j set = +1 in column j).  The reference pins the same two tuples (``rht_constants.py:7-8``; they come from
# the Hadamard tables of the QuaRot tooling, Apache-2.0): a rotated checkpoint is only meaningful with exactly
# these matrices, so they are data of the format, like the nibble order of the packed weights.
HAD12_MASKS = (1, 2955, 1815, 3629, 3163, 2231, 367, 733, 1465, 2929, 1763, 3525)
HAD28_MASKS = (268419071, 185429047, 102422639, 204828893, 141222331, 14009207, 28002029, 55987673, 111958961,
               223901537, 179367619, 90299783, 180583181, 92730907, 16382, 82979893, 165943403, 63484117, 126951851,
               253887319, 239371949, 210341209, 152279729, 36156769, 72297155, 144577927, 20753165, 41489947)
_OFFICIAL_ORDERS = {3072: 12, 14336: 28}
MAX_BLOCK_IN_KERNEL = 256   # longest power-of-two rotation the pre-pass does inside a warp
MAX_PART_IN_KERNEL = 512    # longest power-of-two part of its composite form


def composite_order(width: int) -> int | None:
    """Order of the sign matrix the reference's "rht" rotation uses for this width (``rht.py:31-34``):
    12 at 3072, 28 at 14336, none for powers of two (plain FWHT)."""
    return _OFFICIAL_ORDERS.get(int(width))


@lru_cache(maxsize=None)
def official_hadamard_matrix(order: int) -> torch.Tensor:
    """The order-12 / order-28 matrix of the reference (``rht.py:18-24``) as fp32 +-1 on the CPU."""
    masks = {12: HAD12_MASKS, 28: HAD28_MASKS}[int(order)]
    return torch.tensor([[1.0 if mask >> j & 1 else -1.0 for j in range(order)] for mask in masks])


@lru_cache(maxsize=None)
def sylvester_matrix(order: int) -> torch.Tensor:
    """H_2 x ... x H_2 of a power-of-two order, entry (i, j) = (-1)^popcount(i & j)."""
    if order < 1 or order & (order - 1):
        raise ValueError("Sylvester matrices have power-of-two orders.")
    index = torch.arange(order)
    bits = index[:, None] & index[None, :]
    parity = torch.zeros_like(bits)
    while bool(bits.any()):
        parity ^= bits & 1
        bits = bits >> 1
    return 1.0 - 2.0 * parity.float()


def official_rotation_plan(width: int):
    """How the reference's "rht" rotation of this width (``rht.py:27-39``) maps onto the pre-pass kernel:
    ``("block", width)`` - one power-of-two transform over the whole row, done in a warp - or
    ``("mix", matrix)`` - order x part with ``matrix`` across the parts: had12 x H256 at 3072, had28 x H512 at
    14336, and H_(width/512) x H512 for the powers of two beyond a warp's reach (the same transform: a Sylvester
    matrix factors into Sylvester matrices).  Other widths are refused with the reference's message."""
    width = int(width)
    if width > 0 and width & (width - 1) == 0:
        if width <= MAX_BLOCK_IN_KERNEL:
            return "block", width
        part = min(width // 2, MAX_PART_IN_KERNEL)
        if width // part > 32:
            raise ValueError(f"Official FastWAM RHT of width {width} exceeds what the B200 pre-pass rotates (16384).")
        return "mix", sylvester_matrix(width // part)
    order = _OFFICIAL_ORDERS.get(width)
    if order is None:
        raise ValueError(f"Official FastWAM RHT supports power-of-two widths and 3072/14336, got {width}.")
    return "mix", official_hadamard_matrix(order)


_DEVICE_MATRICES: dict = {}


def official_rotation_matrix(width: int, device) -> torch.Tensor | None:
    """The ``mix`` matrix of ``official_rotation_plan`` on ``device`` (cached per width and device; call once
    outside any CUDA-graph capture), or None when the plan is a plain block transform."""
    kind, what = official_rotation_plan(width)
    if kind == "block":
        return None
    key = (int(width), str(device))
    if key not in _DEVICE_MATRICES:
        _DEVICE_MATRICES[key] = what.to(device=device, dtype=torch.float32).contiguous()
    return _DEVICE_MATRICES[key]


def official_hadamard(values: torch.Tensor) -> torch.Tensor:
    """``_official_hadamard`` of the reference (``rht.py:27-39``), forward direction: full-width normalised FWHT
    for power-of-two widths, had12 / had28 across 256- / 512-long transformed parts at 3072 / 14336."""
    width = int(values.shape[-1])
    if width > 0 and width & (width - 1) == 0:
        return block_hadamard(values, width)
    order = _OFFICIAL_ORDERS.get(width)
    if order is None:
        raise ValueError(f"Official FastWAM RHT supports power-of-two widths and 3072/14336, got {width}.")
    return composite_hadamard(values, official_hadamard_matrix(order))


def randomized_official_hadamard_transform(values: torch.Tensor, signs: torch.Tensor) -> torch.Tensor:
    """``rht_transform(values, signs, "rht")`` of the reference (``rht.py:56-66``)."""
    if values.ndim == 0 or tuple(signs.shape) != (values.shape[-1],):
        raise ValueError("Official RHT requires one sign per input channel.")
    return official_hadamard(values * signs.to(device=values.device, dtype=values.dtype))


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
