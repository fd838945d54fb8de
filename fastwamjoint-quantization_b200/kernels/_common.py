"""Argument checks and dispatch shared by the W4A8 and W4A4 operator modules.

Error behaviour follows the reference: layout / dtype / shape problems found in Python raise
``ValueError`` (``kernels/w4a8/ops.py:17-29``, ``kernels/w4a4/wam_ops.py:10-24``); problems the
reference finds in C++ (an out-of-range schedule index, ``w4a8.cu:1587-1628``) raise ``RuntimeError``.
"""
from __future__ import annotations

import torch

from .. import native

GROUP = 128


def check_common(tag: str, alignment: int, x, packed, scales, bias, inverse):
    if x.dtype not in (torch.bfloat16, torch.float16) or not x.is_cuda or x.ndim < 2:
        raise ValueError(f"{tag} expects CUDA BF16/FP16 inputs with token and channel axes.")
    if packed.ndim != 2:
        raise ValueError("Packed WAM weights must be a two-dimensional tensor.")
    k, n = x.shape[-1], packed.shape[0]
    if packed.dtype != torch.uint8 or packed.shape != (n, k // 2) or k % alignment or n % 8:
        raise ValueError(f"Unsupported FastWAM {tag} shape: K={k}, N={n}.")
    if packed.device != x.device or scales.device != x.device:
        raise ValueError("Packed weights and scales must be on the input device.")
    group = scales.dtype == torch.float16
    if group:
        if k % GROUP or scales.shape != (n, k // GROUP):
            raise ValueError("Group weight scales must be float16 [N, K/128].")
    elif scales.dtype != torch.float32 or scales.shape != (n,):
        raise ValueError("Packed weights and float32 per-channel scales must be on the input device.")
    if inverse is not None and (inverse.dtype != torch.float32 or inverse.device != x.device or inverse.shape != (k,)):
        raise ValueError("Precomputed inverse D must be CUDA float32 [K].")
    if bias is not None and (bias.dtype != x.dtype or bias.device != x.device or bias.shape != (n,)):
        raise ValueError("The native bias must match the input precision and output width.")
    return x.contiguous()


def stream_span(x, gains, token_counts, activation_scales, *, strict_positive: bool):
    """The reference's span encoding (``kernels/w4a8/ops.py:39-51``): equal streams -> positive span,
    a (text, proprio) pair -> minus the proprio count."""
    bad = (gains.ndim != 2 or not token_counts or len(token_counts) != gains.shape[-1]
           or sum(token_counts) != x.shape[-2] or (strict_positive and any(c <= 0 for c in token_counts)))
    if bad:
        raise ValueError("WAM token layout does not match the input and gain schedule.")
    if activation_scales.device != x.device or activation_scales.dtype != torch.float32 or activation_scales.ndim != 1:
        raise ValueError("WAM clipping scale schedule must be CUDA float32 [calls].")
    if gains.device != x.device or gains.dtype != torch.float32 or gains.shape[0] != activation_scales.numel():
        raise ValueError("WAM gains must be CUDA float32 [calls, streams].")
    if len(set(token_counts)) == 1:
        return int(token_counts[0])
    if len(token_counts) == 2 and token_counts[0] > 0 and token_counts[1] > 0:
        return -int(token_counts[1])  # negative span selects the unequal text/proprio layout
    raise ValueError("Native WAM supports equal video/action streams or text/proprio streams.")


def scheduled_linear(x, packed, scales, bias, inverse, activation_scales, gains, span, call, *, abits, signs=None,
                     rht_block=GROUP):
    return native.linear(x, packed, scales, bias, abits=abits, mode="static", inverse=inverse, signs=signs,
                         rht_block=rht_block, act_scales=activation_scales.contiguous(), gains=gains.contiguous(),
                         call=int(call), span=span, streams=gains.shape[-1])


def dynamic_linear(x, packed, scales, bias, inverse, *, abits, signs=None, rht_block=GROUP):
    return native.linear(x, packed, scales, bias, abits=abits, mode="token", inverse=inverse, signs=signs,
                         rht_block=rht_block)
