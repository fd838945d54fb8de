"""Packed deployment files: everything a quantized model needs at run time in one CPU-serializable payload,
with the target Linears stored only as packed int4 (reference: ``deployment.py``, format
``fastwam_steerquant_packed_deployment_v1``).

``export_deployment`` writes the payload from the ORIGINAL model and its calibration checkpoint;
``validate_payload`` is the format's gatekeeper; ``load_deployment`` builds the model without weights
(``meta`` or CPU), puts a ``WAMQuantLinear.from_packed`` at every site and alias, and only then moves to
the GPU - no floating-point target weight ever gets there.  File format, site keys, native-buffer
conventions (``weight`` uint8 [N, K/2], ``input_scale`` = 1/D, ``clipping_ranges`` = clip / qmax) and the
refusals are the reference's, so files written by either side load on the other.
"""
from __future__ import annotations

import json
import os
from pathlib import Path
from typing import Callable

import torch
from torch import nn

from .checkpoint import QuantizationCheckpoint
from .kernels.w4a8.ops import pack_signed_int4
from .runtime import WAMQuantLinear
from .state import DenoiseCallState
from .streams import FastWAMStreamConfig
from .topology import enumerate_fastwamjoint_linears, resolve_site_module, resolve_site_parent

FORMAT = "fastwam_steerquant_packed_deployment_v1"
BUFFERS = ("weight", "weight_scales", "input_scale", "gamma_gains", "clipping_ranges", "bias", "input_rotation_signs")
_POSITIVE_FP32 = ("weight_scales", "input_scale", "gamma_gains", "clipping_ranges")


def _alignment(activation_bits: int) -> int:
    return 256 if activation_bits == 4 else 32


def _host_copy(tensor: torch.Tensor) -> torch.Tensor:
    if tensor.is_meta:
        raise ValueError("Export requires materialized model weights.")
    return tensor.detach().cpu().contiguous()


def registered_paths(model: nn.Module, site_names) -> dict[str, list[str]]:
    """Every path under which each site's Linear is registered (a MoT wrapper may list an expert twice, a model
    may keep a shortcut attribute to one Linear): ``{site name: sorted paths}``."""
    owner: dict[int, str] = {}
    for name in site_names:
        key = id(resolve_site_module(model, name))
        if key in owner:
            raise ValueError("Distinct calibration sites share one Linear; unsupported tying.")
        owner[key] = name
    paths: dict[str, list[str]] = {name: [] for name in site_names}
    for path, module in model.named_modules(remove_duplicate=False):
        name = owner.get(id(module))
        if name is not None:
            paths[name].append(path)
    return {name: sorted(found) for name, found in paths.items()}


def _aliases_of(spec: dict) -> list:
    # files written before aliases existed name only the site itself
    return spec.get("aliases", [spec["module_name"]])


def _native_buffers(entry, source: nn.Linear, activation_bits: int) -> dict:
    """Checkpoint conventions -> the buffers ``WAMQuantLinear`` keeps (``runtime.py:88-92``)."""
    qmax = (1 << (activation_bits - 1)) - 1
    return {
        "weight": pack_signed_int4(entry.qweight.cpu()),
        "weight_scales": entry.weight_scales.float().reshape(-1),
        "input_scale": entry.input_scale.float().reciprocal(),
        "gamma_gains": entry.gamma_gains.float(),
        "clipping_ranges": entry.clipping_ranges.float() / qmax,
        "bias": source.bias,
        "input_rotation_signs": entry.input_rotation_signs,
    }


def _write_once(payload: dict, target: Path) -> None:
    """Durable write-then-rename (the reference routes this through its snapshot helper, ``recovery.py:43-52``)."""
    target.parent.mkdir(parents=True, exist_ok=True)
    scratch = target.with_name(f".{target.name}.{os.getpid()}.tmp")
    with open(scratch, "wb") as handle:
        torch.save(payload, handle)
        handle.flush()
        os.fsync(handle.fileno())
    os.replace(scratch, target)


def export_deployment(model: nn.Module, checkpoint: QuantizationCheckpoint, path: str | Path, *, model_config: dict,
                      provenance: dict | None = None) -> Path:
    """Write a deployment from the original (unrotated, unreplaced) model and its full checkpoint.  Runs wherever
    the model lives (CPU is fine); the model is not modified; the floating-point weights and biases of the target
    Linears are left out of the file (``deployment.py:50-118``)."""
    checkpoint.validate()
    bits = checkpoint.activation_bits
    if checkpoint.weight_bits != 4 or bits not in (4, 8):
        raise ValueError("Deployment requires W4A8 or W4A4 calibration.")
    present = enumerate_fastwamjoint_linears(model)
    if {site.module_name for site in present} != {site.module_name for site in checkpoint.sites}:
        raise ValueError("Export requires calibration of every target Linear, not a partial shard.")
    if any(hasattr(site.module, "_wam_rotation") for site in present):
        raise ValueError("Export requires the original, unrotated model.")
    # through JSON and back: nothing but plain data can reach the file, nothing executes on load
    plain = json.loads(json.dumps({"model_config": model_config, "provenance": provenance or {}}))
    paths = registered_paths(model, [site.module_name for site in checkpoint.sites])
    left_out = {f"{alias}.{leaf}" for found in paths.values() for alias in found for leaf in ("weight", "bias")}
    state = {key: _host_copy(value) for key, value in model.state_dict().items() if key not in left_out}
    specs = []
    for entry in checkpoint.sites:
        source = resolve_site_module(model, entry.module_name)
        n, k = entry.qweight.shape
        if tuple(source.weight.shape) != (n, k):
            raise ValueError(f"Shape mismatch: {entry.module_name}")
        if k % _alignment(bits) or n % 8:
            raise ValueError(f"Unsupported native shape {entry.module_name}: N={n}, K={k}")
        if entry.rotation != "none" and bits != 4:
            raise ValueError("RHT requires W4A4.")
        for leaf, value in _native_buffers(entry, source, bits).items():
            if value is None:
                continue
            shared = _host_copy(value)  # ONE tensor under every alias: torch.save then stores it once
            for alias in paths[entry.module_name]:
                state[f"{alias}.{leaf}"] = shared
        specs.append({"module_name": entry.module_name, "aliases": paths[entry.module_name],
                      "site_index": entry.site_index, "expert": entry.expert, "operation": entry.operation,
                      "stream_names": list(entry.stream_names), "rotation": entry.rotation, "in_features": k,
                      "out_features": n, "has_bias": source.bias is not None})
    # non-persistent buffers (position tables and the like) are not in state_dict; a meta-built model would keep
    # them unmaterialised
    extras = {}
    for prefix, module in model.named_modules():
        for leaf in module._non_persistent_buffers_set:
            value = module._buffers[leaf]
            if value is not None:
                extras[f"{prefix}.{leaf}" if prefix else leaf] = _host_copy(value)
    payload = {"format": FORMAT, "weight_bits": 4, "activation_bits": bits, "num_calls": checkpoint.num_calls,
               "stream_config": checkpoint.stream_config, "sites": specs, "state_dict": state,
               "nonpersistent_buffers": extras, "d_config": checkpoint.d_config,
               "gamma_config": checkpoint.gamma_config, **plain}
    validate_payload(payload)
    target = Path(path).expanduser().resolve()
    if target.exists():
        raise FileExistsError(f"Deployment already exists: {target}")
    _write_once(payload, target)
    return target


def _check_alias_list(spec: dict, taken: set) -> list:
    aliases = _aliases_of(spec)
    well_formed = isinstance(aliases, list) and len(aliases) > 0 and all(
        isinstance(alias, str) and alias and all(alias.split(".")) for alias in aliases)
    if (not well_formed or len(set(aliases)) != len(aliases) or spec["module_name"] not in aliases
            or not taken.isdisjoint(aliases)):
        raise ValueError("Invalid or overlapping deployment aliases.")
    taken.update(aliases)
    return aliases


def _check_site(spec: dict, state: dict, bits: int, calls: int) -> None:
    stem = spec["module_name"] + "."
    n, k, streams = spec["out_features"], spec["in_features"], len(spec["stream_names"])
    if n <= 0 or k <= 0 or k % _alignment(bits) or n % 8 or streams < 1:
        raise ValueError("Unsupported packed deployment shape.")
    weight = state[stem + "weight"]
    if weight.dtype != torch.uint8 or tuple(weight.shape) != (n, k // 2):
        raise ValueError("Deployment weight must be packed uint8 [N,K/2].")
    shapes = {"weight_scales": (n,), "input_scale": (k,), "gamma_gains": (calls, streams), "clipping_ranges": (calls,)}
    for leaf in _POSITIVE_FP32:
        value = state[stem + leaf]
        if value.dtype != torch.float32 or tuple(value.shape) != shapes[leaf]:
            raise ValueError(f"Invalid deployment buffer: {stem}{leaf}")
        if not bool(torch.isfinite(value).all()) or bool((value <= 0).any()):
            raise ValueError(f"Nonpositive/nonfinite deployment scales: {stem}{leaf}")
    bias = state.get(stem + "bias")
    bias_ok = bias is None or (tuple(bias.shape) == (n,) and bias.dtype in (torch.float16, torch.bfloat16))
    if bool(spec["has_bias"]) != (bias is not None) or not bias_ok:
        raise ValueError("Native deployment bias must match model FP16/BF16 precision.")
    rotation, signs = spec["rotation"], state.get(stem + "input_rotation_signs")
    if rotation not in ("none", "rht") or (rotation == "rht" and bits != 4):
        raise ValueError("Invalid deployment RHT mode.")
    if (rotation == "none") != (signs is None):
        raise ValueError("RHT metadata/signs mismatch.")
    if signs is not None and (tuple(signs.shape) != (k,) or signs.dtype != torch.float32
                              or not bool((signs.abs() == 1).all())):
        raise ValueError("Invalid RHT signs.")


def _check_alias_buffers(spec: dict, aliases: list, state: dict) -> None:
    stem = spec["module_name"] + "."
    for alias in aliases:
        for leaf in BUFFERS:
            canonical, copy = state.get(stem + leaf), state.get(f"{alias}.{leaf}")
            if copy is canonical:
                continue
            same = (isinstance(copy, torch.Tensor) and isinstance(canonical, torch.Tensor)
                    and copy.dtype == canonical.dtype and copy.shape == canonical.shape and torch.equal(copy, canonical))
            if not same:
                raise ValueError(f"Conflicting or missing deployment alias buffer: {alias}.{leaf}")


def validate_payload(payload: dict) -> None:
    """Refuse anything that is not a well-formed v1 deployment (``deployment.py:121-177``)."""
    if payload.get("format") != FORMAT or payload.get("weight_bits") != 4:
        raise ValueError("Unsupported deployment format.")
    bits, calls, specs = payload["activation_bits"], payload["num_calls"], payload["sites"]
    if bits not in (4, 8) or calls <= 0 or not specs:
        raise ValueError("Invalid precision, schedule or empty deployment.")
    FastWAMStreamConfig(**payload["stream_config"]).validate()
    if len({spec["module_name"] for spec in specs}) != len(specs):
        raise ValueError("Duplicate deployment sites.")
    taken: set = set()
    for spec in specs:
        aliases = _check_alias_list(spec, taken)
        _check_site(spec, payload["state_dict"], bits, calls)
        _check_alias_buffers(spec, aliases, payload["state_dict"])


def load_deployment(path: str | Path, build_model: Callable, *, device="cuda", construct_device="meta"):
    """``build_model(model_config, device=...)`` must construct the model WITHOUT loading weights.  Returns
    ``(model, DenoiseCallState, metadata)``; the model is on ``device`` in eval mode, every target Linear a native
    ``WAMQuantLinear`` built from the packed buffers (``deployment.py:180-226``)."""
    if construct_device not in ("meta", "cpu"):
        raise ValueError("Construct on meta or CPU to avoid FP GPU allocation.")
    payload = torch.load(Path(path).expanduser(), map_location="cpu", weights_only=True, mmap=True)
    validate_payload(payload)
    model = build_model(payload["model_config"], device=construct_device)
    if any(t.device.type not in ("meta", "cpu") for t in (*model.parameters(), *model.buffers())):
        raise ValueError("Builder placed weights on GPU before packed replacement.")
    present = enumerate_fastwamjoint_linears(model)
    if {site.module_name for site in present} != {spec["module_name"] for spec in payload["sites"]}:
        raise ValueError("Deployment/model topology mismatch.")
    paths = registered_paths(model, [site.module_name for site in present])
    for spec in payload["sites"]:
        if paths[spec["module_name"]] != sorted(_aliases_of(spec)):
            raise ValueError(f"Builder alias topology differs at {spec['module_name']}")
    state = DenoiseCallState(payload["num_calls"])
    stream_config = FastWAMStreamConfig(**payload["stream_config"])
    tensors = payload["state_dict"]
    for spec in payload["sites"]:
        source = resolve_site_module(model, spec["module_name"])
        built = (source.in_features, source.out_features, source.bias is not None)
        if built != (spec["in_features"], spec["out_features"], spec["has_bias"]):
            raise ValueError(f"Builder shape/bias differs at {spec['module_name']}")
        buffers = {leaf: tensors.get(f"{spec['module_name']}.{leaf}") for leaf in BUFFERS}
        packed = WAMQuantLinear.from_packed(spec, buffers, state=state, stream_config=stream_config,
                                            activation_bits=payload["activation_bits"])
        for alias in _aliases_of(spec):
            parent, leaf = resolve_site_parent(model, alias)
            setattr(parent, leaf, packed)
    model.load_state_dict(tensors, strict=True, assign=True)
    for name, value in payload["nonpersistent_buffers"].items():
        prefix, _, leaf = name.rpartition(".")
        holder = resolve_site_module(model, prefix) if prefix else model
        if leaf not in holder._non_persistent_buffers_set:
            raise ValueError(f"Nonpersistent buffer contract changed: {name}")
        holder._buffers[leaf] = value
    if any(t.is_meta for t in (*model.parameters(), *model.buffers())):
        raise ValueError("Builder left unmaterialized buffers; export or rebuild them explicitly.")
    model.to(device=device).eval()
    metadata = {key: value for key, value in payload.items() if key not in ("state_dict", "nonpersistent_buffers")}
    return model, state, metadata
