"""Synthetic DiT stack of the benchmark configurations: 30 blocks, hidden 3072, 24 heads of 128, QKV
3072->9216, attention out 3072->3072, FFN 3072->12288 (GELU) ->3072, RMSNorm, residuals; batch 1 with 1560
latent + 32 action tokens.  Every linear is a ``TokenQuantLinear`` (int4 weights with fp16 group-128 scales,
per-token int8 or int4 activations, optional block-local 128-point rotation); attention stays in bf16
(``scaled_dot_product_attention``).  The reference's model (FastWAMJoint) is not available, so the weights are
random (N(0, 0.02), per-layer seeds) and the stack exists to measure and check one captured denoising step.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import native
from .kernels.w4a8.ops import pack_signed_int4
from .quant import GROUP, quantize_weight_group
from .rht import randomized_block_hadamard_transform, rht_signs, rotate_weight_


class TokenQuantLinear(nn.Module):
    """Group-128 W4 linear with per-token dynamic activations.

    ``backend="native"`` runs the B200 kernels; ``backend="reference"`` is the fake-quant restatement in plain
    torch (rotate -> round to the model dtype -> per-token fake-quant -> ``F.linear`` against the dequantized
    weight), the form the reference's CPU module has (``runtime.py:155-175``).  Both read the same buffers, so
    switching ``backend`` compares like with like."""

    def __init__(self, weight: torch.Tensor, *, activation_bits: int, rotate: bool, module_name: str,
                 bias: torch.Tensor | None = None, backend: str = "native", rotation_seed: int = 0):
        super().__init__()
        n, k = weight.shape
        signs = None
        if rotate:
            signs = rht_signs(k, seed=rotation_seed, module_name=module_name, device=weight.device)
            weight = rotate_weight_(weight.clone(), signs)
        codes, scales = quantize_weight_group(weight.float())
        self.register_buffer("weight", pack_signed_int4(codes))
        self.register_buffer("weight_scales", scales.contiguous())
        self.register_buffer("bias", bias)
        self.register_buffer("input_rotation_signs", signs)
        self.activation_bits, self.backend = int(activation_bits), backend
        self.in_features, self.out_features = k, n
        self._dequantized: torch.Tensor | None = None
        self.workspace: torch.Tensor | None = None  # shared scratch set by the owning stack
        # optional kernel-native copy of the weight (``prepack()``), used from PREPACK_MIN_ROWS input rows on
        self.weight_tiled: torch.Tensor | None = None

    PREPACK_MIN_ROWS = 512  # below this the GEMM is bound by weight bytes, which the unpacked form doubles

    def prepack(self) -> "TokenQuantLinear":
        """Keep a second copy of the weight in the GEMM's operand form (int8 [N, K], ``sq_prepack_weights``):
        the GEMM then skips its unpack stage.  The packed buffer stays the checkpoint format."""
        if self.weight.is_cuda and self.weight_tiled is None:
            self.weight_tiled = native.prepack_weights(self.weight)
        return self

    def _reference_weight(self, dtype):
        if self._dequantized is None or self._dequantized.dtype != dtype:
            low = (self.weight & 0x0F).to(torch.int16)
            high = (self.weight >> 4).to(torch.int16)
            both = torch.stack((low, high), dim=-1).reshape(self.out_features, self.in_features)
            codes = torch.where(both >= 8, both - 16, both).float()
            scales = self.weight_scales.float().repeat_interleave(GROUP, dim=1)
            self._dequantized = (codes * scales).to(dtype)
        return self._dequantized

    def forward(self, x: torch.Tensor, *, rms_eps: float | None = None, input_activation: str | None = None,
                activation: str | None = None, residual: torch.Tensor | None = None) -> torch.Tensor:
        """``residual + act(linear(rms_norm(in_act(x))))`` with every optional part fused into the two kernels
        on the native backend (activated / normalised rows are rounded to x's dtype, as separate modules would)
        and spelled out in torch on the reference backend."""
        if self.backend == "native":
            # the residual add stays a separate elementwise kernel: in the GEMM epilogue it runs on the drain
            # warps, which set the kernel's pace, and measured 20 % slower than GEMM + add
            rows = x.numel() // x.shape[-1]
            weight = self.weight_tiled if self.weight_tiled is not None and rows >= self.PREPACK_MIN_ROWS else self.weight
            y = native.linear(x, weight, self.weight_scales, self.bias, abits=self.activation_bits,
                              mode="token", signs=self.input_rotation_signs, workspace=self.workspace,
                              norm=None if rms_eps is None else "rms", norm_eps=rms_eps or 0.0,
                              round_after_norm=rms_eps is not None, input_activation=input_activation)
            if activation == "gelu":
                y = F.gelu(y)
            return y if residual is None else residual + y
        if input_activation == "gelu":
            x = F.gelu(x)
        if rms_eps is not None:
            x = rms_norm(x, rms_eps)
        y = self._reference_linear(x)
        if activation == "gelu":
            y = F.gelu(y)
        return y if residual is None else residual + y

    @torch.no_grad()
    def input_codes(self, x: torch.Tensor, *, rms_eps: float | None = None, input_activation: str | None = None,
                    backend: str = "native") -> torch.Tensor:
        """The integer activation codes this linear computes for input ``x`` (natural k order), for parity
        diagnostics: the optional GELU / RMSNorm in front are done in torch and rounded to x's dtype for both
        backends, so what is compared is the rotation and the quantizer."""
        if input_activation == "gelu":
            x = F.gelu(x)
        if rms_eps is not None:
            x = rms_norm(x, rms_eps)
        if backend == "native":
            codes, _ = native.prepass(x, abits=self.activation_bits, mode="token", signs=self.input_rotation_signs,
                                      codes_layout=native._lib.CODES_NATURAL)
            return codes.reshape(*x.shape[:-1], self.in_features)
        values = x.float()
        if self.input_rotation_signs is not None:
            values = randomized_block_hadamard_transform(values, self.input_rotation_signs, 128).to(x.dtype).float()
        qmax = (1 << (self.activation_bits - 1)) - 1
        amax = values.abs().amax(dim=-1, keepdim=True)
        scale = (amax / torch.full_like(amax, float(qmax))).clamp_min(1e-8)
        return (values / scale).round().clamp(-qmax, qmax).to(torch.int8)

    def _reference_linear(self, x: torch.Tensor) -> torch.Tensor:
        values = x.float()
        if self.input_rotation_signs is not None:
            values = randomized_block_hadamard_transform(values, self.input_rotation_signs, 128).to(x.dtype).float()
        qmax = (1 << (self.activation_bits - 1)) - 1
        amax = values.abs().amax(dim=-1, keepdim=True)
        # tensor / tensor: on CUDA, torch turns division by a Python scalar into a multiply by its reciprocal,
        # which moves the scale by one ulp and flips int4 codes at rounding ties
        scale = (amax / torch.full_like(amax, float(qmax))).clamp_min(1e-8)
        qx = ((values / scale).round().clamp(-qmax, qmax) * scale).to(x.dtype)
        return F.linear(qx, self._reference_weight(x.dtype), self.bias)


@dataclass(frozen=True)
class DiTConfig:
    blocks: int = 30
    hidden: int = 3072
    heads: int = 24
    ffn: int = 12288
    activation_bits: int = 8
    rotate: bool = False
    latent_tokens: int = 1560
    action_tokens: int = 32
    eps: float = 1e-6

    @property
    def tokens(self) -> int:
        return self.latent_tokens + self.action_tokens


def rms_norm(x: torch.Tensor, eps: float) -> torch.Tensor:
    """RMSNorm with unit weight, fp32 statistics."""
    xf = x.float()
    return (xf * torch.rsqrt(xf.square().mean(dim=-1, keepdim=True) + eps)).to(x.dtype)


class DiTBlock(nn.Module):
    OPERATIONS = ("attn.qkv", "attn.o", "ffn.0", "ffn.2")

    def __init__(self, config: DiTConfig, index: int, device, dtype, backend: str):
        super().__init__()
        self.config = config
        h, f = config.hidden, config.ffn
        shapes = {"attn.qkv": (3 * h, h), "attn.o": (h, h), "ffn.0": (f, h), "ffn.2": (h, f)}
        layers = {}
        for j, op in enumerate(self.OPERATIONS):
            generator = torch.Generator(device=device).manual_seed(1000 + 4 * index + j)
            weight = (torch.randn(shapes[op], generator=generator, device=device) * 0.02).to(dtype)
            layers[op] = TokenQuantLinear(weight, activation_bits=config.activation_bits, rotate=config.rotate,
                                          module_name=f"blocks.{index}.{op}", backend=backend)
        self.qkv, self.o, self.up, self.down = (layers[op] for op in self.OPERATIONS)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        cfg = self.config
        b, m, h = x.shape
        # RMSNorm and GELU ride in the pre-pass of the linear that consumes them (a whole-GPU streaming kernel
        # with ALU to spare); the two residual adds stay elementwise kernels.
        qkv = self.qkv(x, rms_eps=cfg.eps).reshape(b, m, 3, cfg.heads, h // cfg.heads)
        q, k, v = (qkv[:, :, i].transpose(1, 2) for i in range(3))
        attn = F.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(b, m, h)
        x = self.o(attn, residual=x)
        return self.down(self.up(x, rms_eps=cfg.eps), input_activation="gelu", residual=x)


class SyntheticDiT(nn.Module):
    """The stack plus the two hooks the live-graph glue wraps (``_joint_denoise_core``, ``infer_action``)."""

    def __init__(self, config: DiTConfig = DiTConfig(), *, device="cuda", dtype=torch.bfloat16, backend: str = "native"):
        super().__init__()
        self.config = config
        self.blocks = nn.ModuleList(DiTBlock(config, i, device, dtype, backend) for i in range(config.blocks))
        if backend == "native":
            biggest = max(config.hidden, config.ffn)
            lib = native._lib.load_library()
            size = lib.sq_workspace_bytes(config.tokens, biggest) + lib.sq_split_workspace_bytes(config.tokens)
            self.register_buffer("workspace", torch.empty(size, dtype=torch.uint8, device=device), persistent=False)
            for module in self.modules():
                if isinstance(module, TokenQuantLinear):
                    module.workspace = self.workspace

    def prepack(self) -> "SyntheticDiT":
        """Give every linear a kernel-native copy of its weight (see ``TokenQuantLinear.prepack``)."""
        for module in self.modules():
            if isinstance(module, TokenQuantLinear):
                module.prepack()
        return self

    def set_backend(self, backend: str) -> None:
        for module in self.modules():
            if isinstance(module, TokenQuantLinear):
                module.backend = backend

    def forward(self, tokens: torch.Tensor) -> torch.Tensor:
        x = tokens
        for block in self.blocks:
            x = block(x)
        return rms_norm(x, self.config.eps)

    # hooks with the names LiveJointDiTGraph replaces
    def _joint_denoise_core(self, tokens: torch.Tensor):
        return (self.forward(tokens),)

    def infer_action(self, tokens: torch.Tensor, num_inference_steps: int = 1, text_cfg_scale: float = 1.0):
        x = tokens
        for _ in range(num_inference_steps):
            (velocity,) = self._joint_denoise_core(x)
            x = x - velocity / num_inference_steps
        return x


def _rel_fro(a: torch.Tensor, b: torch.Tensor) -> float:
    return float((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-30))


@torch.no_grad()
def stack_parity(model: SyntheticDiT, tokens: torch.Tensor) -> dict:
    """How far the native stack is from its fake-quant reference backend, layer by layer and block by block.

    ``linear``          every linear gets the REFERENCE stack's input of that linear on both backends: relative
                        Frobenius error of its output (largest of the block's four).  This is the kernels' own
                        error, the quantity the 1e-2 output tolerance is about.
    ``code_mismatch``   on the same inputs, the largest fraction of activation codes that differ.
    ``teacher_forced``  every block gets the reference stack's input of that block on both backends: error of the
                        block output.  Inside a block the four linears already feed each other, so this includes
                        how one block of the (random, untrained) stack amplifies a flipped activation code.
    ``free_running``    both stacks run from ``tokens`` on their own: error of the native activations after each block.
    ``output``          the summary, errors after the final norm included.  The reference backend's dequantized
                        weights are freed block by block, so the extra memory is one block's worth."""
    report = {"linear": [], "code_mismatch": [], "teacher_forced": [], "free_running": []}
    reference_x = native_x = tokens
    for block in model.blocks:
        captured = []
        layers = [m for m in block.modules() if isinstance(m, TokenQuantLinear)]
        hooks = [layer.register_forward_pre_hook(lambda mod, args, kwargs: captured.append((mod, args[0], dict(kwargs))),
                                                 with_kwargs=True) for layer in layers]
        for layer in layers:
            layer.backend = "reference"
        reference_out = block(reference_x)
        for hook in hooks:
            hook.remove()
        worst_codes = worst_linear = 0.0
        for layer, x_in, kwargs in captured:
            front = {key: kwargs.get(key) for key in ("rms_eps", "input_activation")}
            ours = layer.input_codes(x_in, backend="native", **front)
            theirs = layer.input_codes(x_in, backend="reference", **front)
            worst_codes = max(worst_codes, float((ours != theirs).float().mean()))
            want = layer(x_in, **kwargs)
            layer.backend = "native"
            worst_linear = max(worst_linear, _rel_fro(layer(x_in, **kwargs), want))
            layer.backend = "reference"
        for layer in layers:
            layer.backend = "native"
            layer._dequantized = None
        report["linear"].append(worst_linear)
        report["code_mismatch"].append(worst_codes)
        report["teacher_forced"].append(_rel_fro(block(reference_x), reference_out))
        native_x = block(native_x)
        report["free_running"].append(_rel_fro(native_x, reference_out))
        reference_x = reference_out
    eps = model.config.eps
    report["output"] = {"linear_max": max(report["linear"]), "code_mismatch_max": max(report["code_mismatch"]),
                        "teacher_forced_max": max(report["teacher_forced"]),
                        "free_running": _rel_fro(rms_norm(native_x, eps), rms_norm(reference_x, eps))}
    return report
