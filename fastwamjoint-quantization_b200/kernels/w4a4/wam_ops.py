"""W4A4 operators with the reference's names and argument order (``kernels/w4a4/wam_ops.py``).

Additions that no reference call site uses: ``symmetric_dynamic_linear`` (per-token int4, optional
rotation), the keyword ``rht_block`` (block length of the local Hadamard rotation, 128 by default) and
float16 ``[N, K/128]`` group scales."""
from __future__ import annotations

import torch

from .._common import (GROUP, adaln_linear, check_common, dynamic_linear, gate_residual_linear, scheduled_linear,
                       stream_span)
from ...rht import official_rotation_matrix, official_rotation_plan
from .loader import load_extension  # noqa: F401


def _common(x, packed, scales, bias, inverse):
    return check_common("W4A4", 256, x, packed, scales, bias, inverse)


def _check_signs(x, signs):
    if signs.shape != (x.shape[-1],) or signs.device != x.device or signs.dtype != torch.float32:
        raise ValueError("Rotation signs must be CUDA float32 [K].")
    return signs.contiguous()


def symmetric_scheduled_stream_linear(x, packed, scales, bias, inverse, activation_scales, gains, token_counts, call):
    """``wam_ops.py:27-45``."""
    x = _common(x, packed, scales, bias, inverse)
    span = stream_span(x, gains, token_counts, activation_scales, strict_positive=True)
    return scheduled_linear(x, packed, scales, bias, inverse, activation_scales, gains, span, call, abits=4)


def symmetric_scheduled_stream_rht_linear(x, packed, scales, bias, inverse, activation_scales, gains, token_counts,
                                          call, signs, *, rht_block: int | None = None, mix=None):
    """Rotate, scale, quantize to int4, multiply (``wam_ops.py:56-75``).  Called as the reference calls it - no
    keyword - the rotation is the reference's for the width (``rht.py:27-39``; device producer
    ``rht.cuh:78-100``): the full-width transform for powers of two, had12 x H256 at K = 3072, had28 x H512 at
    K = 14336, a ``ValueError`` for anything else.  ``rht_block`` opts into a block-local power-of-two transform
    of that length instead, ``mix`` (fp32 ``[order, order]`` sign matrix) into a caller's own composite
    ``order x power of two``.  The first call per width and device caches a small matrix on the device: make it
    outside CUDA-graph capture (the warm-up runs of ``LiveJointDiTGraph`` do)."""
    x = _common(x, packed, scales, bias, inverse)
    span = stream_span(x, gains, token_counts, activation_scales, strict_positive=True)
    if mix is None and rht_block is None:
        kind, what = official_rotation_plan(x.shape[-1])
        if kind == "block":
            rht_block = int(what)
        else:
            mix = official_rotation_matrix(x.shape[-1], x.device)
    if mix is not None:
        return scheduled_linear(x, packed, scales, bias, inverse, activation_scales, gains, span, call, abits=4,
                                signs=_check_signs(x, signs), mix=mix)
    return scheduled_linear(x, packed, scales, bias, inverse, activation_scales, gains, span, call, abits=4,
                            signs=_check_signs(x, signs), rht_block=rht_block)


def symmetric_dynamic_linear(x, packed, scales, bias, inverse, signs=None, *, rht_block: int = GROUP):
    """Per-token dynamic int4 activations (device kernels ``w4a4.cu:918-961`` have no reference wrapper)."""
    x = _common(x, packed, scales, bias, inverse)
    return dynamic_linear(x, packed, scales, bias, inverse, abits=4,
                          signs=None if signs is None else _check_signs(x, signs), rht_block=rht_block)


def symmetric_scheduled_stream_adaln_linear(x, packed, scales, bias, inverse, activation_scales, gains, token_counts,
                                            call, adaln_scale, adaln_shift, epsilon):
    """Affine-free LayerNorm and the MLP AdaLN moved into the activation producer."""
    return adaln_linear("W4A4", 256, 4, x, packed, scales, bias, inverse, activation_scales, gains, token_counts,
                        call, adaln_scale, adaln_shift, epsilon)


def symmetric_scheduled_stream_gate_residual_linear(x, packed, scales, bias, inverse, activation_scales, gains,
                                                    token_counts, call, residual, gate):
    """``x + gate * projection`` moved into the GEMM epilogue."""
    return gate_residual_linear("W4A4", 256, 4, x, packed, scales, bias, inverse, activation_scales, gains,
                                token_counts, call, residual, gate)
