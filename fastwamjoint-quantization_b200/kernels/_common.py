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
    # uint8 [N, K/2]: the checkpoint format; int8 [N, K]: the same weights after native.prepack_weights
    form_ok = ((packed.dtype == torch.uint8 and packed.shape == (n, k // 2))
               or (packed.dtype == torch.int8 and packed.shape == (n, k)))
    if not form_ok or k % alignment or n % 8:
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
                     rht_block=GROUP, **fused):
    # `call` is the reference's Python int, or a one-element CUDA int32 tensor read when the kernels run
    index = call if isinstance(call, torch.Tensor) else None
    return native.linear(x, packed, scales, bias, abits=abits, mode="static", inverse=inverse, signs=signs,
                         rht_block=rht_block, act_scales=activation_scales.contiguous(), gains=gains.contiguous(),
                         call=0 if index is not None else int(call), call_index=index, span=span,
                         streams=gains.shape[-1], **fused)


def equal_stream_span(x, gains, token_counts, tag: str) -> int:
    """The fused entries need equal-length streams (``kernels/w4a8/ops.py:58-63``)."""
    if (gains.ndim != 2 or not token_counts or any(c <= 0 for c in token_counts)
            or len(token_counts) != gains.shape[-1] or sum(token_counts) != x.shape[-2]):
        raise ValueError("WAM fused stream layout does not cover the input token axis.")
    if len(set(token_counts)) != 1:
        raise ValueError(f"The fused {tag} producer requires equal-length FastWAM streams.")
    return int(token_counts[0])


def adaln_linear(tag, alignment, abits, x, packed, scales, bias, inverse, activation_scales, gains, token_counts, call,
                 adaln_scale, adaln_shift, epsilon):
    """Affine-free LayerNorm and AdaLN ``(1 + scale) * x_hat + shift`` folded into the pre-pass
    (``kernels/w4a8/ops.py:66-84``, device side ``w4a8.cu:615-691``)."""
    x = check_common(tag, alignment, x, packed, scales, bias, inverse)
    span = equal_stream_span(x, gains, token_counts, tag)
    if (adaln_scale.shape != adaln_shift.shape or adaln_scale.shape[-1] != x.shape[-1] or adaln_scale.dtype != x.dtype
            or adaln_scale.device != x.device or adaln_shift.dtype != x.dtype or adaln_shift.device != x.device):
        raise ValueError("AdaLN scale and shift must match the input dtype and hidden width.")
    rows = x.numel() // x.shape[-1]
    modulation_rows = adaln_scale.numel() // x.shape[-1]
    if modulation_rows <= 0 or rows % modulation_rows:
        raise ValueError("AdaLN groups must cover complete input rows.")
    return scheduled_linear(x, packed, scales, bias, inverse, activation_scales, gains, span, call, abits=abits,
                            norm="layer", norm_eps=float(epsilon), mod_scale=adaln_scale, mod_shift=adaln_shift)


def gate_residual_linear(tag, alignment, abits, x, packed, scales, bias, inverse, activation_scales, gains,
                         token_counts, call, residual, gate):
    """``residual + gate * projection`` folded into the GEMM epilogue (``kernels/w4a8/ops.py:87-105``,
    device side ``w4a8.cu:383-479``)."""
    x = check_common(tag, alignment, x, packed, scales, bias, inverse)
    span = equal_stream_span(x, gains, token_counts, tag)
    n = packed.shape[0]
    if residual.shape != (*x.shape[:-1], n) or residual.dtype != x.dtype or residual.device != x.device:
        raise ValueError("Residual must match the projection output shape and dtype.")
    if gate.dtype != x.dtype or gate.device != x.device or gate.shape[-1] != n:
        raise ValueError("Gate must match the projection output dtype and width.")
    rows = x.numel() // x.shape[-1]
    gate_rows = gate.numel() // n
    if gate_rows <= 0 or rows % gate_rows:
        raise ValueError("Gate groups must cover complete output rows.")
    return scheduled_linear(x, packed, scales, bias, inverse, activation_scales, gains, span, call, abits=abits,
                            residual=residual, gate=gate)


def dynamic_linear(x, packed, scales, bias, inverse, *, abits, signs=None, rht_block=GROUP):
    return native.linear(x, packed, scales, bias, abits=abits, mode="token", inverse=inverse, signs=signs,
                         rht_block=rht_block)
