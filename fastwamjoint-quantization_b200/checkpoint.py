"""The per-site record a calibrated checkpoint holds (reference: ``checkpoint.py:15-70``).  Only the
dataclass and its validation are mirrored here; calibration itself is outside the hot path."""
from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class QuantizedSite:
    site_index: int
    module_name: str
    expert: str
    operation: str
    stream_names: tuple[str, ...]
    qweight: torch.Tensor          # int8 [N, K] in [-8, 7]
    weight_scales: torch.Tensor    # fp32 [N, 1]
    input_scale: torch.Tensor      # D, fp32 [K]
    gamma_gains: torch.Tensor      # fp32 [calls, streams]
    clipping_ranges: torch.Tensor  # clip, fp32 [calls]
    token_fractions: torch.Tensor  # fp32 [calls, streams]
    d_initial_loss: float = 0.0
    d_final_loss: float = 0.0
    gamma_initial_losses: tuple[float, ...] = ()
    gamma_final_losses: tuple[float, ...] = ()
    input_rotation_signs: torch.Tensor | None = None
    rotation: str = "none"

    def validate(self, num_calls: int) -> None:
        if self.qweight.ndim != 2 or self.qweight.dtype != torch.int8:
            raise ValueError("qweight must be a two-dimensional int8 tensor.")
        n, k = self.qweight.shape
        if self.rotation not in ("none", "rht"):
            raise ValueError("Unsupported WAM checkpoint rotation.")
        signs = self.input_rotation_signs
        if (signs is None) != (self.rotation == "none"):
            raise ValueError("WAM rotation metadata/signs do not match.")
        if signs is not None and (signs.shape != (k,) or not torch.all(signs.abs() == 1)):
            raise ValueError("WAM rotation signs must be finite +/-1 per input channel.")
        streams = len(self.stream_names)
        if streams == 0 or len(set(self.stream_names)) != streams:
            raise ValueError("stream_names must be non-empty and unique.")
        if self.weight_scales.shape != (n, 1):
            raise ValueError("weight_scales must be per output channel.")
        if self.input_scale.shape != (k,):
            raise ValueError("input_scale shape does not match qweight.")
        if self.gamma_gains.shape != (num_calls, streams):
            raise ValueError("gamma_gains has an invalid shape.")
        if self.clipping_ranges.shape != (num_calls,):
            raise ValueError("clipping_ranges has an invalid shape.")
        if self.token_fractions.shape != self.gamma_gains.shape:
            raise ValueError("token_fractions must match gamma_gains.")
        for value in (self.weight_scales, self.input_scale, self.gamma_gains, self.clipping_ranges):
            if not torch.isfinite(value).all() or (value <= 0).any():
                raise ValueError("Checkpoint scales, gains, and clips must be finite and positive.")
        fractions = self.token_fractions
        if not torch.isfinite(fractions).all() or (fractions < 0).any():
            raise ValueError("token_fractions must be finite and non-negative.")
        if not torch.allclose(fractions.sum(dim=1), torch.ones(num_calls), atol=1e-6, rtol=0):
            raise ValueError("token_fractions must sum to one per call.")
