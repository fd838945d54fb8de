"""W4A8 operators with the reference's names and argument order (``kernels/w4a8/ops.py``), running on
the B200 kernels.  ``scales`` may also be float16 ``[N, K/128]`` (group-128 weight scales); every
reference call site passes float32 ``[N]`` and behaves as before."""
from __future__ import annotations

import torch

from .._common import adaln_linear, check_common, dynamic_linear, gate_residual_linear, scheduled_linear, stream_span
from .loader import load_extension  # noqa: F401  (part of the reference's surface)


def pack_signed_int4(qweight: torch.Tensor) -> torch.Tensor:
    """int8 [N, even K] in [-8, 7] -> uint8 [N, K/2], low nibble = even k (``ops.py:8-14``)."""
    if qweight.ndim != 2 or qweight.dtype != torch.int8 or qweight.shape[-1] % 2:
        raise ValueError("W4A8 expects INT8 [N, even K] weights containing signed INT4 values.")
    if not qweight.is_cuda and qweight.numel() and (qweight.min() < -8 or qweight.max() > 7):
        raise ValueError("Quantized weights must lie in [-8, 7].")
    nibble = qweight.to(torch.uint8) & 0x0F
    return (nibble[:, ::2] | (nibble[:, 1::2] << 4)).contiguous()


def _common(x, packed, scales, bias, inverse):
    return check_common("W4A8", 32, x, packed, scales, bias, inverse)


def symmetric_dynamic_linear(x, packed, scales, bias, inverse):
    """Per-token dynamic int8 activations (``ops.py:32-34``, ``w4a8.cu:693-747``)."""
    x = _common(x, packed, scales, bias, inverse)
    return dynamic_linear(x, packed, scales, bias, inverse, abits=8)


def symmetric_scheduled_stream_linear(x, packed, scales, bias, inverse, activation_scales, gains, token_counts, call):
    """Static per-call scale and per-stream gain (``ops.py:37-55``)."""
    x = _common(x, packed, scales, bias, inverse)
    span = stream_span(x, gains, token_counts, activation_scales, strict_positive=False)
    return scheduled_linear(x, packed, scales, bias, inverse, activation_scales, gains, span, call, abits=8)


def symmetric_scheduled_stream_adaln_linear(x, packed, scales, bias, inverse, activation_scales, gains, token_counts,
                                            call, adaln_scale, adaln_shift, epsilon):
    """Affine-free LayerNorm and the MLP AdaLN moved into the activation producer."""
    return adaln_linear("W4A8", 32, 8, x, packed, scales, bias, inverse, activation_scales, gains, token_counts,
                        call, adaln_scale, adaln_shift, epsilon)


def symmetric_scheduled_stream_gate_residual_linear(x, packed, scales, bias, inverse, activation_scales, gains,
                                                    token_counts, call, residual, gate):
    """``x + gate * projection`` moved into the GEMM epilogue."""
    return gate_residual_linear("W4A8", 32, 8, x, packed, scales, bias, inverse, activation_scales, gains,
                                token_counts, call, residual, gate)
