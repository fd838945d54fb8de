"""``WAMQuantLinear``: the reference's quantized Linear (``runtime.py:15-276``) on the B200 kernels.

Same constructor, buffers, backend strings and errors as the reference, so code written against
``fastwam_steerquant.runtime`` keeps working:

* ``backend="reference"`` is the fake-quant forward in plain torch (``runtime.py:155-175``); it runs on
  any device and is what the native path is compared with.
* ``backend="cutlass_w4a8"`` / ``"cutlass_w4a4"`` keep their names (they are part of checkpoints and
  call sites) but dispatch to the hand-written sm_100a kernels; nothing here is CUTLASS.

Native buffers follow the deployment conventions (``runtime.py:88-92``, ``deployment.py:89-91``):
``weight`` packed uint8 [N, K/2], ``weight_scales`` fp32 [N], ``input_scale`` = 1/D, ``clipping_ranges`` =
clip / qmax, ``gamma_gains`` [calls, streams], optional ``input_rotation_signs`` fp32 [K].

Rotated sites (``rotation == "rht"``) use the reference's rotation for their width (``rht.py:27-39``): the
full-width transform for powers of two, had12 x H256 at K = 3072, had28 x H512 at K = 14336; any other width
is refused, as the reference refuses it.  ``rotation_block`` (a block-local power-of-two transform) and
``rotation_matrix`` (a caller's own order x power-of-two composite) are explicit opt-ins for checkpoints that
were rotated that way; nothing selects them by default.
"""
from __future__ import annotations

from typing import Literal

import torch
import torch.nn as nn
import torch.nn.functional as F

from .checkpoint import QuantizedSite
from .quant import symmetric_fake_quant
from .rht import (official_rotation_plan, randomized_block_hadamard_transform, randomized_composite_hadamard_transform,
                  randomized_official_hadamard_transform)
from .state import DenoiseCallState
from .streams import FastWAMStreamConfig, expand_stream_gains, resolve_stream_layout
from .topology import LinearSite, resolve_site_module, resolve_site_parent, stream_kind_of

BACKENDS = ("reference", "cutlass_w4a8", "cutlass_w4a4")
_BUFFERS = ("weight", "weight_scales", "input_scale", "gamma_gains", "clipping_ranges", "bias", "input_rotation_signs")
# "rotation_matrix" is an optional extra buffer of rotated sites (see the module docstring)


def resolve_rotation(width: int, rotation_block, rotation_matrix):
    """(block, matrix) a rotated site of this width hands to the kernels.  With neither opt-in given this is the
    reference's rotation for the width (``official_rotation_plan``); widths it does not cover raise."""
    if rotation_matrix is not None:
        return 0, rotation_matrix
    if rotation_block:
        return int(rotation_block), None
    kind, what = official_rotation_plan(width)
    return (int(what), None) if kind == "block" else (0, what.clone())


def _native_ops(activation_bits: int):
    if activation_bits == 4:
        from .kernels.w4a4 import wam_ops as ops
    else:
        from .kernels.w4a8 import ops
    return ops


class WAMQuantLinear(nn.Module):
    """Reference or native W4A8 / W4A4 Linear with static D and per-stream gains."""

    @classmethod
    def from_packed(cls, spec: dict, tensors: dict, *, state: DenoiseCallState, stream_config: FastWAMStreamConfig,
                    activation_bits: int):
        """Build a native Linear straight from deployment buffers, no floating-point weight involved
        (``runtime.py:18-47``)."""
        if activation_bits not in (4, 8):
            raise ValueError("Deployment supports W4A4 or W4A8.")
        rotation = spec["rotation"]
        if rotation not in ("none", "rht") or (rotation != "none" and activation_bits != 4):
            raise ValueError("RHT deployment requires W4A4.")
        self = cls.__new__(cls)
        nn.Module.__init__(self)
        self.backend = f"cutlass_w4a{activation_bits}"
        self._native_ops = _native_ops(activation_bits)
        self.state, self.stream_config = state, stream_config
        self.weight_bits, self.activation_bits = 4, activation_bits
        self.rotation = rotation
        self.stream_names = tuple(spec["stream_names"])
        self.supports_fused_adaln = False
        self.supports_fused_gate_residual = False
        for name in _BUFFERS:
            self.register_buffer(name, tensors.get(name))
        self.official_rotation = False
        self.rotation_block, matrix = 0, None
        if rotation != "none":
            self.official_rotation = not spec.get("rotation_block") and tensors.get("rotation_matrix") is None
            self.rotation_block, matrix = resolve_rotation(self.weight.shape[1] * 2, spec.get("rotation_block"),
                                                           tensors.get("rotation_matrix"))
            if matrix is not None and self.weight.device.type != "meta":  # a meta build keeps it on the CPU until .to()
                matrix = matrix.float().to(self.weight.device)
        self.register_buffer("rotation_matrix", matrix, persistent=False)
        self.site = LinearSite(spec["site_index"], spec["expert"], -1, spec["operation"], spec["module_name"], None,
                               stream_kind_of(spec["operation"]))
        return self

    def __init__(self, source: nn.Linear, entry: QuantizedSite, *, state: DenoiseCallState,
                 stream_config: FastWAMStreamConfig, weight_bits: int, activation_bits: int,
                 backend: Literal["reference", "cutlass_w4a8", "cutlass_w4a4"] = "reference",
                 fuse_block: bool = False, rotation_block: int | None = None,
                 rotation_matrix: torch.Tensor | None = None) -> None:
        super().__init__()
        entry.validate(state.num_calls)
        if backend not in BACKENDS:
            raise ValueError(f"Unsupported WAM backend: {backend}.")
        native = backend != "reference"
        if native and (weight_bits != 4 or activation_bits != (4 if backend == "cutlass_w4a4" else 8)):
            raise ValueError(f"WAM {backend} does not match W{weight_bits}A{activation_bits}.")
        rotated = entry.rotation != "none"
        if rotated and backend == "cutlass_w4a8":
            raise ValueError("Rotated WAM requires reference or cutlass_w4a4.")
        if rotated and fuse_block:
            raise ValueError("Rotated FastWAM block fusion is not validated; leave fuse_block=False.")
        device = source.weight.device
        qmax = (1 << (activation_bits - 1)) - 1
        self.rotation = entry.rotation
        self.official_rotation = rotated and not rotation_block and rotation_matrix is None
        signs = entry.input_rotation_signs
        self.register_buffer("input_rotation_signs", None if signs is None else signs.float().to(device))
        if rotation_matrix is not None:
            order = int(rotation_matrix.shape[0])
            width = int(entry.qweight.shape[1])
            part = width // order if order > 0 and width % order == 0 else 0
            if (not rotated or rotation_matrix.ndim != 2 or rotation_matrix.shape[1] != order or part < 8
                    or part > 512 or part & (part - 1)):
                raise ValueError("rotation_matrix must be a square sign matrix whose order times a power of two "
                                 "(8..512) is the input width of a rotated site.")
        self.rotation_block = 0
        if rotated:
            self.rotation_block, rotation_matrix = resolve_rotation(entry.qweight.shape[1], rotation_block, rotation_matrix)
        if rotation_matrix is not None:
            rotation_matrix = rotation_matrix.float().to(device)
        # derived from the width (or given by the caller): not part of the state dict, whose keys stay the reference's
        self.register_buffer("rotation_matrix", rotation_matrix, persistent=False)
        if native:
            ops = _native_ops(activation_bits)
            self._native_ops = ops
            from .kernels.w4a8 import pack_signed_int4
            self.register_buffer("weight", pack_signed_int4(entry.qweight).to(device))
            self.register_buffer("weight_scales", entry.weight_scales.float().reshape(-1).to(device))
            self.register_buffer("input_scale", entry.input_scale.float().reciprocal().to(device))
            self.register_buffer("gamma_gains", entry.gamma_gains.float().to(device))
            self.register_buffer("clipping_ranges", (entry.clipping_ranges.float() / qmax).to(device))
        else:
            dtype = source.weight.dtype
            # dequantize once at load instead of at every call (runtime.py:94-98)
            self.register_buffer("weight", entry.qweight.to(device=device, dtype=dtype)
                                 * entry.weight_scales.to(device=device, dtype=dtype))
            self.register_buffer("weight_scales", None)
            self.register_buffer("input_scale", entry.input_scale.clone())
            self.register_buffer("gamma_gains", entry.gamma_gains.clone())
            self.register_buffer("clipping_ranges", entry.clipping_ranges.clone())
        self.register_buffer("bias", None if source.bias is None else source.bias.detach().clone())
        self.state, self.stream_config = state, stream_config
        self.weight_bits, self.activation_bits = int(weight_bits), int(activation_bits)
        self.backend = backend
        self.stream_names = entry.stream_names
        self.supports_fused_adaln = bool(fuse_block and native and entry.operation == "ffn.0")
        self.supports_fused_gate_residual = bool(fuse_block and native and entry.operation in {"self_attn.o", "ffn.2"})
        # the replaced bf16 Linear is deliberately not kept (it would stay resident on the GPU)
        self.site = LinearSite(entry.site_index, entry.expert, -1, entry.operation, entry.module_name, None,
                               stream_kind_of(entry.operation))

    @property
    def in_features(self) -> int:
        return self.weight.shape[1] * (1 if self.backend == "reference" else 2)

    @property
    def out_features(self) -> int:
        return self.weight.shape[0]

    def _layout(self, x: torch.Tensor, what: str):
        layout = resolve_stream_layout(self.site, x.shape[-2], self.stream_config)
        if self.backend != "reference" and layout.names != self.stream_names:
            raise RuntimeError(f"WAM {what} stream names differ from {self.site.module_name}: {layout.names}.")
        return layout

    def prepack(self) -> "WAMQuantLinear":
        """Native backends: keep a second copy of the weight in the GEMM's operand form (int8 [N, K],
        ``sq_prepack_weights``), made from the packed checkpoint-format buffer, which stays as it is
        (deployment files keep their v1 format, ``deployment.py:180-226``).  The GEMM then skips its unpack
        stage.  Call after the module is on its GPU."""
        if self.backend != "reference" and self.weight.is_cuda:
            from . import native
            self._weight_tiled = native.prepack_weights(self.weight.contiguous())
        return self

    PREPACK_MIN_ROWS = 512  # below this the GEMM is bound by weight bytes, which the unpacked form doubles

    def _native_weight(self, rows: int | None = None) -> torch.Tensor:
        """The packed checkpoint-format weight, or its kernel-native copy when there is one and the call has
        enough input rows for the GEMM to be compute-bound."""
        tiled = getattr(self, "_weight_tiled", None)
        if tiled is None or tiled.device != self.weight.device:
            return self.weight
        if rows is not None and rows < self.PREPACK_MIN_ROWS:
            return self.weight
        return tiled

    def _call(self, x: torch.Tensor):
        """The active call for a native launch: the Python index, or - when the state is ``on_device`` - the
        state's device tensor, which the kernels read when they run (one graph for all calls)."""
        call = self.state.require()
        if getattr(self.state, "on_device", False):
            return self.state.device_index(x.device)
        return call

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        call = self.state.require()
        layout = self._layout(x, "checkpoint")
        if self.backend != "reference":
            call = self._call(x)
            args = (x, self._native_weight(x.numel() // x.shape[-1]), self.weight_scales, self.bias, self.input_scale, self.clipping_ranges,
                    self.gamma_gains, layout.token_counts, call)
            if self.input_rotation_signs is not None:
                return self._native_ops.symmetric_scheduled_stream_rht_linear(
                    *args, self.input_rotation_signs, rht_block=self.rotation_block, mix=self.rotation_matrix)
            return self._native_ops.symmetric_scheduled_stream_linear(*args)
        return self._reference_forward(x, call, layout)

    def _reference_forward(self, x, call, layout):
        """Fake-quant forward of the reference (``runtime.py:155-175``), dividing order."""
        if self.input_rotation_signs is not None and self.official_rotation:
            # rht_transform(x.float(), signs, "rht").to(x.dtype): the reference's own arithmetic (runtime.py:156-157)
            x = randomized_official_hadamard_transform(x.float(), self.input_rotation_signs.to(x.device)).to(x.dtype)
        elif self.input_rotation_signs is not None and self.rotation_matrix is not None:
            x = randomized_composite_hadamard_transform(x.float(), self.input_rotation_signs, self.rotation_matrix).to(x.dtype)
        elif self.input_rotation_signs is not None:
            x = randomized_block_hadamard_transform(x.float(), self.input_rotation_signs, self.rotation_block).to(x.dtype)
        gains = self.gamma_gains[call].to(device=x.device, dtype=torch.float32)
        if gains.numel() != layout.num_streams:
            raise RuntimeError(f"Runtime stream count changed for {self.site.module_name}: "
                               f"checkpoint={gains.numel()}, input={layout.num_streams}.")
        scaled = x.float() / self.input_scale.to(x.device)[None, :]
        row_gain = expand_stream_gains(scaled, gains, layout)
        clip = self.clipping_ranges[call].to(x.device)
        # tensor / tensor keeps IEEE division on CUDA too (a Python-scalar divisor becomes a reciprocal multiply)
        step = clip / torch.full_like(clip, float((1 << (self.activation_bits - 1)) - 1))
        qx = (symmetric_fake_quant(scaled * row_gain, bits=self.activation_bits, scale=step) / row_gain).to(x.dtype)
        bias = None if self.bias is None else self.bias.to(device=x.device, dtype=x.dtype)
        return F.linear(qx, self.weight, bias)

    def forward_adaln(self, x, scale, shift, epsilon: float):
        if not self.supports_fused_adaln:
            raise RuntimeError("WAM AdaLN block fusion was not enabled for this site.")
        layout = self._layout(x, "fused AdaLN")
        return self._native_ops.symmetric_scheduled_stream_adaln_linear(
            x, self._native_weight(x.numel() // x.shape[-1]), self.weight_scales, self.bias, self.input_scale, self.clipping_ranges, self.gamma_gains,
            layout.token_counts, self._call(x), scale, shift, epsilon)

    def forward_gate_residual(self, x, residual, gate):
        if not self.supports_fused_gate_residual:
            raise RuntimeError("WAM gate/residual block fusion was not enabled for this site.")
        layout = self._layout(x, "fused residual")
        return self._native_ops.symmetric_scheduled_stream_gate_residual_linear(
            x, self._native_weight(x.numel() // x.shape[-1]), self.weight_scales, self.bias, self.input_scale, self.clipping_ranges, self.gamma_gains,
            layout.token_counts, self._call(x), residual, gate)


def set_wam_block_fusions(model: nn.Module, enabled: bool) -> int:
    """Toggle the three fusable operations per expert block (``runtime.py:208-223``)."""
    if getattr(model, "_rollout_graph", None) is not None:
        raise RuntimeError("Cannot change block fusion after CUDA Graph installation.")
    modules = [m for m in model.modules() if isinstance(m, WAMQuantLinear)]
    if enabled and any(m.rotation != "none" for m in modules):
        raise ValueError("Rotated FastWAM block fusion is not validated.")
    count = 0
    for module in modules:
        if module.backend == "reference":
            continue
        module.supports_fused_adaln = bool(enabled and module.site.operation == "ffn.0")
        module.supports_fused_gate_residual = bool(enabled and module.site.operation in {"self_attn.o", "ffn.2"})
        count += int(module.supports_fused_adaln or module.supports_fused_gate_residual)
    return count


def apply_checkpoint(model: nn.Module, checkpoint, *, state: DenoiseCallState | None = None,
                     backend: Literal["reference", "cutlass_w4a8", "cutlass_w4a4"] = "reference",
                     fuse_block: bool = False, prepack: bool = False):
    """Replace every site's ``nn.Linear`` by a ``WAMQuantLinear`` (``runtime.py:226-276``).  ``prepack`` also
    gives every native site on a GPU its kernel-native weight copy (``WAMQuantLinear.prepack``).  ``checkpoint``
    needs ``validate()``, ``sites``, ``weight_bits``, ``activation_bits``, ``num_calls`` and
    ``stream_config`` like the reference's ``QuantizationCheckpoint``.  All sites are validated before the
    first replacement; replacement is one site at a time so no second copy of the model exists."""
    checkpoint.validate()
    rotated = any(site.rotation != "none" for site in checkpoint.sites)
    if rotated and (fuse_block or backend == "cutlass_w4a8"):
        raise ValueError("Rotated WAM requires W4A4/reference with block fusion disabled.")
    if backend not in BACKENDS:
        raise ValueError(f"Unsupported WAM backend: {backend}.")
    if backend != "reference" and (checkpoint.weight_bits != 4 or backend != f"cutlass_w4a{checkpoint.activation_bits}"):
        raise ValueError("WAM native backend and checkpoint bit widths must match.")
    state = DenoiseCallState(checkpoint.num_calls) if state is None else state
    if state.num_calls != checkpoint.num_calls:
        raise ValueError("Runtime call state and checkpoint call counts differ.")
    stream_config = FastWAMStreamConfig(**checkpoint.stream_config)
    alignment = 256 if backend == "cutlass_w4a4" else 32
    for entry in checkpoint.sites:
        module = resolve_site_module(model, entry.module_name)
        if not isinstance(module, nn.Linear):
            raise TypeError(f"{entry.module_name} is not an nn.Linear.")
        if module.weight.shape != entry.qweight.shape:
            raise ValueError(f"WAM checkpoint shape differs from {entry.module_name}.")
        if backend != "reference" and (module.in_features % alignment or module.out_features % 8):
            raise ValueError(f"Unsupported {backend} shape at {entry.module_name}.")
    for entry in checkpoint.sites:
        module = resolve_site_module(model, entry.module_name)
        parent, child = resolve_site_parent(model, entry.module_name)
        replacement = WAMQuantLinear(module, entry, state=state, stream_config=stream_config,
                                     weight_bits=checkpoint.weight_bits, activation_bits=checkpoint.activation_bits,
                                     backend=backend, fuse_block=fuse_block).to(module.weight.device)
        replacement.train(module.training)
        if prepack:
            replacement.prepack()
        setattr(parent, child, replacement)
    return state, len(checkpoint.sites)
