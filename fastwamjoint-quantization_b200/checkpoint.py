"""What a calibrated checkpoint holds: the per-site record (reference: ``checkpoint.py:15-70``) and the
container with its two on-disk formats (``checkpoint.py:72-221``).  Calibration itself, which produces these
tensors, is outside the hot path; the container is here because ``apply_checkpoint`` and the packed-deployment
export consume it."""
from __future__ import annotations

import os
from dataclasses import dataclass, fields
from pathlib import Path
from typing import Any, Iterable

import torch

FORMAT = "fastwam_steerquant_calibration_v1"
ROTATED_FORMAT = "fastwam_steerquant_calibration_rht_v1"


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


_SITE_TENSORS = {"qweight": torch.int8, "weight_scales": torch.float32, "input_scale": torch.float32,
                 "gamma_gains": torch.float32, "clipping_ranges": torch.float32, "token_fractions": torch.float32,
                 "input_rotation_signs": torch.float32}
_CONFIG_KEYS = ("weight_bits", "activation_bits", "num_calls", "stream_config", "d_config", "gamma_config")


def _site_record(site: QuantizedSite) -> dict[str, Any]:
    record = {}
    for f in fields(site):
        value = getattr(site, f.name)
        record[f.name] = value.cpu() if isinstance(value, torch.Tensor) else value
    return record


def _site_from_record(record: dict[str, Any]) -> QuantizedSite:
    tensors = {name: (None if record.get(name) is None else torch.as_tensor(record[name], dtype=dtype).cpu())
               for name, dtype in _SITE_TENSORS.items()}
    return QuantizedSite(
        site_index=int(record["site_index"]), module_name=str(record["module_name"]), expert=str(record["expert"]),
        operation=str(record["operation"]), stream_names=tuple(record["stream_names"]),
        d_initial_loss=float(record["d_initial_loss"]), d_final_loss=float(record["d_final_loss"]),
        gamma_initial_losses=tuple(float(v) for v in record["gamma_initial_losses"]),
        gamma_final_losses=tuple(float(v) for v in record["gamma_final_losses"]),
        rotation=str(record.get("rotation", "none")), **tensors)


@dataclass(frozen=True)
class QuantizationCheckpoint:
    """All calibrated sites of one model plus the settings they were calibrated under.  Same fields, formats
    (``fastwam_steerquant_calibration_v1`` / ``..._rht_v1``) and refusals as the reference's container."""

    weight_bits: int
    activation_bits: int
    num_calls: int
    stream_config: dict[str, Any]
    d_config: dict[str, Any]
    gamma_config: dict[str, Any]
    sites: tuple[QuantizedSite, ...]

    @property
    def rotated(self) -> bool:
        return bool(self.sites) and self.sites[0].rotation != "none"

    def validate(self) -> None:
        for bits in (self.weight_bits, self.activation_bits):
            if not 2 <= bits <= 8:
                raise ValueError("Checkpoint bit widths must be in [2, 8].")
        if self.num_calls <= 0 or not self.sites:
            raise ValueError("Checkpoint needs at least one call and site.")
        if len({site.module_name for site in self.sites}) != len(self.sites):
            raise ValueError("Checkpoint module names must be unique.")
        for site in self.sites:
            site.validate(self.num_calls)
        if any(site.rotation != self.sites[0].rotation for site in self.sites):
            raise ValueError("Cannot mix rotated and unrotated WAM sites.")

    def _config(self) -> tuple:
        return tuple(getattr(self, key) for key in _CONFIG_KEYS)

    def state_dict(self) -> dict[str, Any]:
        self.validate()
        payload = {"format": ROTATED_FORMAT if self.rotated else FORMAT}
        payload.update(zip(_CONFIG_KEYS, self._config()))
        payload["sites"] = [_site_record(site) for site in self.sites]
        return payload

    @classmethod
    def from_state_dict(cls, payload: dict[str, Any]) -> "QuantizationCheckpoint":
        if payload.get("format") not in (FORMAT, ROTATED_FORMAT):
            raise ValueError(f"Expected checkpoint format {FORMAT!r} or {ROTATED_FORMAT!r}.")
        loaded = cls(int(payload["weight_bits"]), int(payload["activation_bits"]), int(payload["num_calls"]),
                     dict(payload["stream_config"]), dict(payload["d_config"]), dict(payload["gamma_config"]),
                     tuple(_site_from_record(record) for record in payload["sites"]))
        loaded.validate()
        if loaded.rotated != (payload["format"] == ROTATED_FORMAT):
            raise ValueError("Checkpoint format and rotation metadata disagree.")
        return loaded

    @classmethod
    def merge(cls, checkpoints: Iterable["QuantizationCheckpoint"]) -> "QuantizationCheckpoint":
        """Join shards calibrated separately (disjoint site indices, identical settings)."""
        shards = tuple(checkpoints)
        if not shards:
            raise ValueError("At least one quantization checkpoint is required.")
        for shard in shards:
            shard.validate()
            if shard._config() != shards[0]._config():
                raise ValueError("Quantization checkpoint configurations do not match.")
        sites = sorted((site for shard in shards for site in shard.sites), key=lambda site: site.site_index)
        if len({site.site_index for site in sites}) != len(sites):
            raise ValueError("Quantization checkpoint shards overlap.")
        merged = cls(*shards[0]._config(), tuple(sites))
        merged.validate()
        return merged

    def save(self, path: str | Path) -> Path:
        """Write next to the target and rename, so a reader never meets a half-written file."""
        target = Path(path).expanduser().resolve()
        target.parent.mkdir(parents=True, exist_ok=True)
        scratch = target.with_name(f".{target.name}.{os.getpid()}.tmp")
        torch.save(self.state_dict(), scratch)
        os.replace(scratch, target)
        return target

    @classmethod
    def load(cls, path: str | Path) -> "QuantizationCheckpoint":
        return cls.from_state_dict(torch.load(Path(path).expanduser(), map_location="cpu", weights_only=True))
