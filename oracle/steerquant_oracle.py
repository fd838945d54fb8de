"""CPU oracle for the SteerQuant quantized-linear path.  TEST INFRASTRUCTURE ONLY.

This module restates, in plain torch-on-CPU arithmetic, what the reference
(CathyyW/Fastwamjoint-quantization, package ``fastwam_steerquant``) computes on
its CPU fake-quant path for one quantized linear.  It is the checker the CUDA
path is compared against.  It is never imported by the product package: only
the tests, the smoke entry and the CPU-baseline leg of the benchmark may use it.

Parity status: PINNED.  Every primitive below is checked against outputs of the
reference itself (``tests/golden/steerquant_golden.npz``, written by
``tests/golden/make_golden.py`` which imports the reference package) and
against the seeded generators of the reference's own GPU tests
(``tests/test_wam_w4a4.py:17-36``, ``tests/test_w4a8.py:13-29``,
``tests/test_rht.py:126-132``), which need no fixture file.

Two quantization schemes are covered:

* ``static``  - the reference's production scheme: per-output-channel fp32
  weight scales, a per-channel migration vector ``1/D``, a per-call activation
  scale and a per-stream gain (``runtime.py:155-175`` for the dividing CPU
  module, ``w4a8.cu:838-881`` / ``tests/test_wam_w4a4.py:32-36`` for the
  multiplying kernel order).
* ``token``   - the benchmark scheme: group-128 int4 weights with fp16 scales,
  per-token dynamic activation scales, optional block-local 128-point
  randomized Hadamard transform.  The reference has no single function for it;
  it is composed here from the reference's own primitives
  (``quant.py:6-21,55-64``, ``rht.py:81-112``, ``rht_install.py:39-49``).

Integer results (codes, accumulators) are exact; accumulators are produced with
float64 matrix products, which are exact for these magnitudes (|acc| < 2**53),
the same device the reference's own exact test uses
(``tests/test_wam_w4a4.py:32-36``).
"""
from __future__ import annotations

import hashlib
import math

import torch
import torch.nn.functional as F

GROUP = 128  # weight-scale group length along K in the ``token`` scheme
RHT_BLOCK = 128  # block length of the local Hadamard transform in the ``token`` scheme


# ----------------------------------------------------------------------------
# int4 packing  (reference: kernels/w4a8/ops.py:8-14)
# ----------------------------------------------------------------------------
def pack_signed_int4(qweight: torch.Tensor) -> torch.Tensor:
    """int8 [N, K] in [-8, 7] -> uint8 [N, K/2]; low nibble = even k, high nibble = odd k."""
    if qweight.ndim != 2 or qweight.dtype != torch.int8 or qweight.shape[-1] % 2:
        raise ValueError("expects INT8 [N, even K] weights containing signed INT4 values.")
    if qweight.numel() and (qweight.min() < -8 or qweight.max() > 7):
        raise ValueError("Quantized weights must lie in [-8, 7].")
    nibble = qweight.to(torch.uint8) & 0x0F
    return (nibble[:, ::2] | (nibble[:, 1::2] << 4)).contiguous()


def unpack_signed_int4(packed: torch.Tensor) -> torch.Tensor:
    """Inverse of :func:`pack_signed_int4` (two's-complement nibbles)."""
    low = (packed & 0x0F).to(torch.int16)
    high = (packed >> 4).to(torch.int16)
    both = torch.stack((low, high), dim=-1).reshape(*packed.shape[:-1], packed.shape[-1] * 2)
    return torch.where(both >= 8, both - 16, both).to(torch.int8)


# ----------------------------------------------------------------------------
# weights  (reference: quant.py:55-64)
# ----------------------------------------------------------------------------
def quantize_weight_per_channel(weight: torch.Tensor, *, bits: int = 4):
    """Per-output-channel symmetric quantization, exactly ``quant.py:55-64``."""
    fp32 = weight.detach().float()
    qmax = 2 ** (int(bits) - 1) - 1
    scales = fp32.abs().amax(dim=1, keepdim=True).clamp_min(1e-8) / qmax
    qweight = (fp32 / scales).round().clamp(-qmax, qmax).to(torch.int8)
    return qweight, scales


def quantize_weight_group(weight: torch.Tensor, *, bits: int = 4, group: int = GROUP):
    """Group-wise symmetric quantization along K.

    ``quant.py:55-64`` applied to ``weight.reshape(N*K/group, group)``; the scale
    is rounded to fp16 (the storage type the benchmark configuration names)
    *before* the codes are computed, so codes and stored scales are consistent.
    Returns ``(qweight int8 [N, K], scales fp16 [N, K/group])``.
    """
    n, k = weight.shape
    if k % group:
        raise ValueError("K must be a multiple of the group length.")
    fp32 = weight.detach().float().reshape(n * (k // group), group)
    qmax = 2 ** (int(bits) - 1) - 1
    scales = (fp32.abs().amax(dim=1, keepdim=True).clamp_min(1e-8) / qmax).half()
    scales = scales.clamp_min(torch.finfo(torch.float16).tiny)
    qweight = (fp32 / scales.float()).round().clamp(-qmax, qmax).to(torch.int8)
    return qweight.reshape(n, k), scales.reshape(n, k // group)


# ----------------------------------------------------------------------------
# randomized Hadamard transform  (reference: rht.py:81-112, rht.py:119-123)
# ----------------------------------------------------------------------------
def rht_signs(in_features: int, *, seed: int, module_name: str) -> torch.Tensor:
    """Seeded +/-1 vector, exactly ``rht.py:81-96``."""
    digest = hashlib.sha256(f"{int(seed)}:{module_name}".encode()).digest()
    local_seed = int.from_bytes(digest[:8], "little") % (2**63 - 1)
    generator = torch.Generator(device="cpu").manual_seed(local_seed)
    signs = torch.randint(0, 2, (int(in_features),), generator=generator, dtype=torch.int8)
    return signs.mul_(2).sub_(1).float()


def block_hadamard(values: torch.Tensor, block: int = RHT_BLOCK) -> torch.Tensor:
    """Normalised Sylvester-order FWHT over consecutive ``block``-long pieces of
    the last axis.  Follows ``rht.py:99-112`` (butterfly strides 1, 2, 4, ...
    in that order, one final multiply by ``1/sqrt(block)``); the reference
    derives the block from the width, here it is explicit, which is the same as
    calling the reference on ``values.reshape(..., K/block, block)``.
    """
    width = int(values.shape[-1])
    if block <= 0 or block & (block - 1) or width % block:
        raise ValueError("block must be a power of two dividing the width.")
    work = values.float().reshape(-1, width // block, block).clone()
    butterfly = 1
    while butterfly < block:
        paired = work.reshape(-1, width // block, block // (2 * butterfly), 2, butterfly)
        left = paired[..., 0, :].clone()
        right = paired[..., 1, :].clone()
        paired[..., 0, :] = left + right
        paired[..., 1, :] = left - right
        butterfly *= 2
    return work.reshape(values.shape) * (1.0 / math.sqrt(block))


def rht_rotate(values: torch.Tensor, signs: torch.Tensor, block: int = RHT_BLOCK) -> torch.Tensor:
    """``block_hadamard(values * signs)`` in fp32 (``rht.py:119-123``)."""
    return block_hadamard(values.float() * signs.float(), block)


def composite_hadamard(values: torch.Tensor, matrix: torch.Tensor) -> torch.Tensor:
    """The rotation of widths that are ``order x power of two`` (3072 = 12 x 256, 14336 = 28 x 512), following
    ``rht.py:27-39``: view the last axis as ``[order, P]``, normalised FWHT of length P on every row, then the
    ``order x order`` sign matrix applied across the rows, then one division by ``sqrt(order)``.  The reference
    rebuilds its order-12 / order-28 matrices from pinned masks (``rht.py:18-24``); here the matrix is an argument."""
    order = int(matrix.shape[0])
    width = int(values.shape[-1])
    if matrix.shape != (order, order) or width % order:
        raise ValueError("matrix must be square and its order must divide the width.")
    part = width // order
    if part & (part - 1):
        raise ValueError("width / order must be a power of two.")
    blocks = values.float().reshape(-1, order, part)
    transformed = block_hadamard(blocks, part)
    return (matrix.float() @ transformed).reshape(values.shape) / math.sqrt(order)


def composite_rotate(values: torch.Tensor, signs: torch.Tensor, matrix: torch.Tensor) -> torch.Tensor:
    """``composite_hadamard(values * signs)`` in fp32 (``rht.py:45-46``)."""
    return composite_hadamard(values.float() * signs.float(), matrix)


# Row masks of the reference's order-12 / order-28 sign matrices (bit j set = +1 in column j), as pinned in
# ``rht_constants.py:7-8``; checked against matrices recorded from the reference (``tests/golden``).
_HAD12_MASKS = (1, 2955, 1815, 3629, 3163, 2231, 367, 733, 1465, 2929, 1763, 3525)
_HAD28_MASKS = (268419071, 185429047, 102422639, 204828893, 141222331, 14009207, 28002029, 55987673, 111958961,
                223901537, 179367619, 90299783, 180583181, 92730907, 16382, 82979893, 165943403, 63484117, 126951851,
                253887319, 239371949, 210341209, 152279729, 36156769, 72297155, 144577927, 20753165, 41489947)


def official_matrix(order: int) -> torch.Tensor:
    """``official_hadamard_matrix`` (``rht.py:18-24``)."""
    masks = {12: _HAD12_MASKS, 28: _HAD28_MASKS}[order]
    return torch.tensor([[1.0 if mask & (1 << j) else -1.0 for j in range(order)] for mask in masks])


def official_rotate(values: torch.Tensor, signs: torch.Tensor) -> torch.Tensor:
    """``rht_transform(values, signs, "rht")`` (``rht.py:27-39, 45-46, 61-63``): the width picks the transform -
    one full-width normalised FWHT for a power of two, had12 x H256 at 3072, had28 x H512 at 14336."""
    width = int(values.shape[-1])
    signed = values.float() * signs.float()
    if width > 0 and width & (width - 1) == 0:
        return block_hadamard(signed, width)
    if width not in (3072, 14336):
        raise ValueError(f"Official FastWAM RHT supports power-of-two widths and 3072/14336, got {width}.")
    return composite_hadamard(signed, official_matrix(12 if width == 3072 else 28))


def rotate_weight(weight: torch.Tensor, signs: torch.Tensor, dtype: torch.dtype,
                  block: int = RHT_BLOCK) -> torch.Tensor:
    """Weight-side rotation: fp32 rotate, round to the model dtype
    (``rht_install.py:39-41``)."""
    return rht_rotate(weight.float(), signs, block).to(dtype)


# ----------------------------------------------------------------------------
# activations
# ----------------------------------------------------------------------------
def symmetric_fake_quant(values: torch.Tensor, *, bits: int, scale: torch.Tensor) -> torch.Tensor:
    """Exactly ``quant.py:6-21`` without the straight-through branch."""
    qmax = 2 ** (int(bits) - 1) - 1
    normalized = values / scale.clamp_min(1e-8)
    return normalized.round().clamp(-qmax, qmax) * scale


def token_codes(x: torch.Tensor, *, bits: int, signs: torch.Tensor | None = None,
                inverse: torch.Tensor | None = None, block: int = RHT_BLOCK):
    """Per-token dynamic activation codes of the ``token`` scheme.

    x (bf16/fp16 [..., M, K]) -> optional RHT in fp32, rounded to x's dtype and
    back (the ``rht_fp32_to_model_v1`` contract, ``rht_install.py:20,46-49``)
    -> optional multiply by ``inverse`` (1/D, ``runtime.py:90``) -> per-row
    absmax -> ``scale = amax / qmax`` -> the arithmetic of ``quant.py:15-21``
    (divide by ``scale.clamp_min(1e-8)``, round half to even, clamp).
    Returns ``(codes int8 [..., M, K], row_scales fp32 [..., M])`` where
    ``row_scales`` is the clamped scale actually divided by.
    """
    qmax = 2 ** (int(bits) - 1) - 1
    values = x.float()
    if signs is not None:
        values = rht_rotate(values, signs, block).to(x.dtype).float()
    if inverse is not None:
        values = values * inverse.float()
    amax = values.abs().amax(dim=-1, keepdim=True)
    scale = (amax / qmax).clamp_min(1e-8)
    codes = (values / scale).round().clamp(-qmax, qmax).to(torch.int8)
    return codes, scale.squeeze(-1)


def stream_rows(values: torch.Tensor, token_counts) -> torch.Tensor:
    """Expand one value per stream to one value per token row
    (``streams.py:104-120``)."""
    return torch.repeat_interleave(values, torch.tensor(list(token_counts)))


def static_codes(x: torch.Tensor, *, bits: int, inverse: torch.Tensor,
                 activation_scales: torch.Tensor, gains: torch.Tensor, token_counts, call: int,
                 signs: torch.Tensor | None = None, block: int = RHT_BLOCK):
    """Static-schedule activation codes in the *kernel* operation order
    (``w4a8.cu:838-881``; ``tests/test_wam_w4a4.py:32-36``;
    ``tests/test_rht.py:126-132`` for the rotated form):
    ``code = clamp(round(x * inverse * (gain / scale)))``, ``row_scale = scale / gain``.
    Returns ``(codes int8 [..., M, K], row_scales fp32 [M])``.
    """
    qmax = 2 ** (int(bits) - 1) - 1
    values = x.float()
    if signs is not None:
        values = rht_rotate(values, signs, block).to(x.dtype).float()
    gain = stream_rows(gains[call].float(), token_counts)
    scale = activation_scales[call].float()
    gain_over_scale = (gain / scale)[:, None]
    codes = (values * inverse.float() * gain_over_scale).round().clamp(-qmax, qmax).to(torch.int8)
    return codes, scale / gain


# ----------------------------------------------------------------------------
# integer contraction and epilogue
# ----------------------------------------------------------------------------
def group_accumulators(codes: torch.Tensor, qweight: torch.Tensor, group: int | None = GROUP) -> torch.Tensor:
    """Exact integer accumulators ``acc[m, n, g] = sum_{k in group g} a[m,k] * w[n,k]``
    as int64 (the device holds the same numbers as int32).  ``group=None``
    sums over all of K (one group).  Exact through float64
    (``tests/test_wam_w4a4.py:35``)."""
    m, k = codes.shape[-2:]
    n = qweight.shape[0]
    group = k if group is None else group
    a = codes.reshape(-1, k // group, group).double().permute(1, 0, 2)  # [G, M', group]
    w = qweight.reshape(n, k // group, group).double().permute(1, 2, 0)  # [G, group, N]
    acc = torch.bmm(a, w)  # [G, M', N]
    return acc.permute(1, 2, 0).round().to(torch.int64).reshape(*codes.shape[:-1], n, k // group)


def epilogue_group(acc: torch.Tensor, weight_scales: torch.Tensor, row_scales: torch.Tensor,
                   bias: torch.Tensor | None, dtype: torch.dtype) -> torch.Tensor:
    """``out = dtype( (sum_g float(acc_g) * s_w[n, g]) * s_x[m] + bias[n] )`` in fp32,
    groups added in ascending order (group form of ``w4a8.cu:324-360``)."""
    total = torch.zeros(acc.shape[:-1], dtype=torch.float32)
    scales = weight_scales.float()
    for g in range(acc.shape[-1]):
        total = total + acc[..., g].float() * scales[:, g]
    total = total * row_scales.float().reshape(*row_scales.shape, 1)
    if bias is not None:
        total = total + bias.float()
    return total.to(dtype)


def epilogue_channel(acc: torch.Tensor, weight_scales: torch.Tensor, row_scales: torch.Tensor,
                     bias: torch.Tensor | None, dtype: torch.dtype) -> torch.Tensor:
    """``out = dtype( (float(acc) * row_scale[m]) * w_scale[n] + bias[n] )``
    (``w4a8.cu:324-360``; ``tests/test_wam_w4a4.py:36``)."""
    total = acc.float() * row_scales.float().reshape(-1, 1) * weight_scales.float().reshape(-1)
    if bias is not None:
        total = total + bias.float()
    return total.to(dtype)


# ----------------------------------------------------------------------------
# whole linears
# ----------------------------------------------------------------------------
def linear_token(x: torch.Tensor, qweight: torch.Tensor, weight_scales: torch.Tensor,
                 bias: torch.Tensor | None, *, abits: int, signs: torch.Tensor | None = None,
                 inverse: torch.Tensor | None = None, group: int = GROUP,
                 want_accumulators: bool = True) -> dict:
    """One ``token``-scheme linear.  Returns codes, row scales, the per-group
    integer accumulators and the output in x's dtype."""
    codes, row_scales = token_codes(x, bits=abits, signs=signs, inverse=inverse)
    flat = codes.reshape(-1, codes.shape[-1])
    acc = group_accumulators(flat, qweight, group)
    out = epilogue_group(acc, weight_scales, row_scales.reshape(-1), bias, x.dtype)
    result = {"codes": codes, "row_scales": row_scales,
              "out": out.reshape(*x.shape[:-1], qweight.shape[0])}
    if want_accumulators:
        result["acc"] = acc
    return result


def linear_static(x: torch.Tensor, qweight: torch.Tensor, weight_scales: torch.Tensor,
                  bias: torch.Tensor | None, inverse: torch.Tensor, activation_scales: torch.Tensor,
                  gains: torch.Tensor, token_counts, call: int, *, abits: int,
                  signs: torch.Tensor | None = None, block: int = RHT_BLOCK) -> dict:
    """One ``static``-scheme linear in the kernel operation order, the oracle the
    reference's own GPU tests use (``tests/test_wam_w4a4.py:32-36``)."""
    codes, row_scales = static_codes(x, bits=abits, inverse=inverse, activation_scales=activation_scales,
                                     gains=gains, token_counts=token_counts, call=call, signs=signs,
                                     block=block)
    batch = x.numel() // (x.shape[-1] * x.shape[-2])
    rows = row_scales.repeat(batch)
    flat = codes.reshape(-1, codes.shape[-1])
    acc = group_accumulators(flat, qweight, None)[..., 0]
    out = epilogue_channel(acc, weight_scales, rows, bias, x.dtype)
    return {"codes": codes, "row_scales": rows, "acc": acc,
            "out": out.reshape(*x.shape[:-1], qweight.shape[0])}


def reference_module_forward(x: torch.Tensor, qweight: torch.Tensor, weight_scales: torch.Tensor,
                             bias: torch.Tensor | None, input_scale: torch.Tensor,
                             clipping_ranges: torch.Tensor, gamma_gains: torch.Tensor, token_counts,
                             call: int, *, abits: int, signs: torch.Tensor | None = None,
                             block: int | None = None) -> torch.Tensor:
    """The reference CPU module, ``WAMQuantLinear(backend="reference").forward``
    (``runtime.py:155-175``): optional rotation rounded to x's dtype, divide by D,
    multiply by the row gain, fake-quantize with ``clip / qmax``, divide by the
    gain, cast, ``F.linear`` against the dequantized weight in x's dtype
    (``runtime.py:94-98``).  ``input_scale`` is D and ``clipping_ranges`` the
    clip, i.e. checkpoint conventions, not the native-buffer ones.
    ``block=None`` rotates over the reference's own block (largest power of two
    dividing K, ``rht.py:69-78``)."""
    dtype = x.dtype
    weight = qweight.to(dtype) * weight_scales.reshape(-1, 1).to(dtype)
    if signs is not None:
        k = x.shape[-1]
        x = rht_rotate(x.float(), signs, (k & -k) if block is None else block).to(dtype)
    x_prime = x.float() / input_scale.float()[None, :]
    gain = stream_rows(gamma_gains[call].float(), token_counts)
    shape = [1] * x.ndim
    shape[-2] = x.shape[-2]
    expanded = gain.reshape(shape)
    scale = clipping_ranges[call].float() / (2 ** (abits - 1) - 1)
    qx = (symmetric_fake_quant(x_prime * expanded, bits=abits, scale=scale) / expanded).to(dtype)
    return F.linear(qx, weight, None if bias is None else bias.to(dtype))


def token_module_forward(x: torch.Tensor, qweight: torch.Tensor, weight_scales: torch.Tensor,
                         bias: torch.Tensor | None, *, abits: int, signs: torch.Tensor | None = None,
                         group: int = GROUP) -> torch.Tensor:
    """Fake-quant form of the ``token`` scheme, shaped like the reference CPU
    module (``runtime.py:155-175``): dequantized weight in x's dtype, fake-quantized
    activation in x's dtype, one ``F.linear``.  This is what the reference would
    run on CPU for this scheme and is the timed CPU baseline; it is *not* integer
    exact (bf16 products) and is only compared at the 1e-2 level."""
    dtype = x.dtype
    n, k = qweight.shape
    weight = (qweight.reshape(n, k // group, group).float()
              * weight_scales.float().reshape(n, k // group, 1)).reshape(n, k).to(dtype)
    values = x.float()
    if signs is not None:
        values = rht_rotate(values, signs).to(dtype).float()
    qmax = 2 ** (abits - 1) - 1
    scale = values.abs().amax(dim=-1, keepdim=True) / qmax
    qx = symmetric_fake_quant(values, bits=abits, scale=scale).to(dtype)
    return F.linear(qx, weight, None if bias is None else bias.to(dtype))


# ----------------------------------------------------------------------------
# seeded synthetic inputs of the benchmark configurations
# ----------------------------------------------------------------------------
def synthetic_linear(m: int, k: int, n: int, *, seed: int = 0, x_seed: int | None = None,
                     dtype: torch.dtype = torch.bfloat16, outlier_fraction: float = 0.01,
                     outlier_gain: float = 20.0):
    """Weights N(0, 0.02), activations N(0, 1) with a seeded 1 % of channels scaled x20.
    Draw order: W, X, channel permutation (all from one CPU generator), unless
    ``x_seed`` is given, in which case X and the permutation come from a second
    generator seeded with it (used by the M sweep so W is shared)."""
    gen = torch.Generator(device="cpu").manual_seed(int(seed))
    w = torch.randn(n, k, generator=gen) * 0.02
    gx = gen if x_seed is None else torch.Generator(device="cpu").manual_seed(int(x_seed))
    x = torch.randn(m, k, generator=gx)
    count = int(math.ceil(outlier_fraction * k))
    idx = torch.randperm(k, generator=gx)[:count]
    x[:, idx] *= outlier_gain
    return w, x.to(dtype)


def prepare_token_linear(m: int, k: int, n: int, *, abits: int, seed: int = 0, x_seed: int | None = None,
                         module_name: str = "linear", dtype: torch.dtype = torch.bfloat16) -> dict:
    """Everything one ``token``-scheme linear needs: x, int4 codes of the
    (optionally rotated) weight, fp16 group scales, zero bias, signs."""
    w, x = synthetic_linear(m, k, n, seed=seed, x_seed=x_seed, dtype=dtype)
    signs = None
    if abits == 4:
        signs = rht_signs(k, seed=0, module_name=module_name)
        w = rotate_weight(w, signs, dtype).float()
    qweight, scales = quantize_weight_group(w)
    return {"x": x, "qweight": qweight, "weight_scales": scales,
            "bias": torch.zeros(n, dtype=dtype), "signs": signs, "abits": abits}
