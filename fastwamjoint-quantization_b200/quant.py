"""Host-side quantization helpers (torch; CPU or CUDA tensors).  Same names and arithmetic as the
reference's ``quant.py``; ``quantize_weight_group`` adds the group-128 / fp16-scale form the
benchmark configurations use.  These run once at load time, not on the hot path."""
from __future__ import annotations

import torch

GROUP = 128


def _qmax(bits: int) -> int:
    bits = int(bits)
    if not 2 <= bits <= 8:
        raise ValueError("bits must be in [2, 8].")
    return (1 << (bits - 1)) - 1


def symmetric_fake_quant(values: torch.Tensor, *, bits: int, scale: torch.Tensor, ste: bool = False) -> torch.Tensor:
    """Quantize-dequantize on a symmetric grid (``quant.py:6-21``): divide by ``scale`` (floored at 1e-8),
    round half to even, clamp to +-qmax, multiply back.  ``ste`` keeps the gradient of the identity."""
    limit = _qmax(bits)
    ratio = values / scale.clamp_min(1e-8)
    snapped = ratio.round()
    if ste:
        snapped = ratio + (snapped - ratio).detach()
    return snapped.clamp(-limit, limit) * scale


def fake_quant_activation_per_tensor(values: torch.Tensor, *, bits: int, clipping_range=None, ste: bool = False):
    """Per-tensor activation fake-quant with an explicit or observed clip (``quant.py:24-40``)."""
    work = values.float()
    if clipping_range is None:
        clip = work.detach().abs().amax()
    else:
        clip = torch.as_tensor(clipping_range, device=work.device, dtype=torch.float32)
    if clip.numel() != 1 or not torch.isfinite(clip) or clip <= 0:
        raise ValueError("clipping_range must be one finite positive scalar.")
    return symmetric_fake_quant(work, bits=bits, scale=clip.reshape(()) / _qmax(bits), ste=ste).to(values.dtype)


def fake_quant_weight_per_channel(weight: torch.Tensor, *, bits: int, ste: bool = False) -> torch.Tensor:
    """``quant.py:43-52``."""
    work = weight.float()
    scales = work.detach().abs().amax(dim=1, keepdim=True).clamp_min(1e-8) / _qmax(bits)
    return symmetric_fake_quant(work, bits=bits, scale=scales, ste=ste).to(weight.dtype)


def quantize_weight_per_channel(weight: torch.Tensor, *, bits: int):
    """int8 codes and fp32 ``[N, 1]`` scales, one scale per output channel (``quant.py:55-64``)."""
    work = weight.detach().float()
    limit = _qmax(bits)
    scales = work.abs().amax(dim=1, keepdim=True).clamp_min(1e-8) / limit
    codes = (work / scales).round().clamp(-limit, limit).to(torch.int8)
    return codes, scales


def quantize_weight_group(weight: torch.Tensor, *, bits: int = 4, group: int = GROUP):
    """int8 codes ``[N, K]`` and fp16 scales ``[N, K/group]``: the per-channel rule applied to each run of
    ``group`` input channels, with the scale rounded to fp16 before the codes are computed."""
    n, k = weight.shape
    if k % group:
        raise ValueError("K must be a multiple of the group length.")
    limit = _qmax(bits)
    rows = weight.detach().float().reshape(n * (k // group), group)
    scales = (rows.abs().amax(dim=1, keepdim=True).clamp_min(1e-8) / limit).half()
    scales = scales.clamp_min(torch.finfo(torch.float16).tiny)
    codes = (rows / scales.float()).round().clamp(-limit, limit).to(torch.int8)
    return codes.reshape(n, k), scales.reshape(n, k // group)
