"""Tensor-level wrappers over the C ABI: they allocate outputs and scratch with
``torch.empty`` on the current device (so CUDA-graph capture uses PyTorch's
graph-private pool, as the reference's ``torch::empty`` calls do,
``kernels/w4a8/csrc/w4a8.cu:1358-1360``) and launch on the current stream."""
from __future__ import annotations

import torch

from . import _lib

_DTYPES = {torch.bfloat16: _lib.BF16, torch.float16: _lib.FP16}


def _require_cuda(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor: the B200 path has no CPU fallback.")


def _ptr(t):
    return None if t is None else t.data_ptr()


def _stream():
    return torch.cuda.current_stream().cuda_stream


def prepass(x: torch.Tensor, *, abits: int, mode: str, inverse=None, signs=None, rht_block: int = 128,
            act_scale=None, gains=None, span: int = 1, streams: int = 1, seq_tokens: int | None = None,
            codes_layout: int = _lib.CODES_EVEN_ODD, pack_int4: bool = False, out=None, mix=None):
    """Run the fused activation pre-pass.  ``x`` is [..., tokens, K] bf16/fp16.
    Returns ``(codes, row_scales)``: int8 [rows, K] (or uint8 [rows, K/2] when
    ``pack_int4``) and fp32 [rows].  ``mix`` (fp32 [order, order] of +-1) selects the composite rotation
    ``order x power of two`` instead of the block rotation of length ``rht_block``."""
    _require_cuda(x, "x")
    x = x.contiguous()
    k = x.shape[-1]
    rows = x.numel() // k
    if out is not None:
        codes, row_scales = out
    else:
        codes = torch.empty((rows, k // 2) if pack_int4 else (rows, k), device=x.device,
                            dtype=torch.uint8 if pack_int4 else torch.int8)
        row_scales = torch.empty((rows,), device=x.device, dtype=torch.float32)
    if mix is not None:
        mix = _mix_matrix(mix, x)
        with torch.cuda.device(x.device):
            status = _lib.load_library().sq_prepass_composite(
                x.data_ptr(), _DTYPES[x.dtype], rows, k, int(abits),
                _lib.ACT_TOKEN if mode == "token" else _lib.ACT_STATIC,
                _ptr(inverse), _ptr(signs), mix.data_ptr(), int(mix.shape[0]), _ptr(act_scale), _ptr(gains),
                int(span), int(streams), int(seq_tokens if seq_tokens is not None else x.shape[-2]),
                int(codes_layout), int(bool(pack_int4)), codes.data_ptr(), row_scales.data_ptr(), _stream())
        _lib.check(status, "sq_prepass_composite")
        return codes, row_scales
    with torch.cuda.device(x.device):
        status = _lib.load_library().sq_prepass(
            x.data_ptr(), _DTYPES[x.dtype], rows, k, int(abits),
            _lib.ACT_TOKEN if mode == "token" else _lib.ACT_STATIC,
            _ptr(inverse), _ptr(signs), int(rht_block), _ptr(act_scale), _ptr(gains),
            int(span), int(streams), int(seq_tokens if seq_tokens is not None else x.shape[-2]),
            int(codes_layout), int(bool(pack_int4)), codes.data_ptr(), row_scales.data_ptr(), _stream())
    _lib.check(status, "sq_prepass")
    return codes, row_scales


def prepack_weights(packed: torch.Tensor) -> torch.Tensor:
    """uint8 [N, K/2] packed int4 weights -> int8 [N, K] in the GEMM's own operand form (``sq_prepack_weights``).
    Pass the result wherever ``packed`` goes: ``gemm`` and ``linear`` tell the two forms apart by dtype."""
    _require_cuda(packed, "packed")
    if packed.dtype != torch.uint8 or packed.ndim != 2 or not packed.is_contiguous():
        raise ValueError("packed must be a contiguous uint8 [N, K/2] tensor.")
    n, half = packed.shape
    tiled = torch.empty((n, 2 * half), device=packed.device, dtype=torch.int8)
    with torch.cuda.device(packed.device):
        status = _lib.load_library().sq_prepack_weights(packed.data_ptr(), n, 2 * half, tiled.data_ptr(), _stream())
    _lib.check(status, "sq_prepack_weights")
    return tiled


def _wscale_mode(packed: torch.Tensor, w_scales: torch.Tensor) -> int:
    mode = _lib.WSCALE_GROUP_F16 if w_scales.dtype == torch.float16 else _lib.WSCALE_CHANNEL_F32
    return mode | (_lib.WEIGHTS_PREPACKED if packed.dtype == torch.int8 else 0)


def _mix_matrix(mix: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    if mix.ndim != 2 or mix.shape[0] != mix.shape[1] or mix.dtype != torch.float32 or mix.device != x.device:
        raise ValueError("mix must be a square fp32 matrix on the input's device.")
    return mix.contiguous()


def gemm(codes: torch.Tensor, packed: torch.Tensor, w_scales: torch.Tensor, row_scales: torch.Tensor, bias,
         *, out_dtype: torch.dtype, codes_layout: int = _lib.CODES_EVEN_ODD, want_accumulators: bool = False,
         check_kernel: bool = False, out: torch.Tensor | None = None, int4_range: bool = False,
         split: bool = True):
    """codes int8 [M, K] x packed uint8 [N, K/2] -> [M, N] in ``out_dtype``.
    ``w_scales`` fp32 [N] selects the per-channel form, fp16 [N, K/128] the group form.
    ``int4_range`` promises that every code lies in [-8, 7] (SQ_CODES_INT4_RANGE): faster group form.
    ``check_kernel`` runs the CUDA-core cross-check kernel instead of the tensor-core one (tests only).
    ``split`` lends the kernel scratch for tiles split along K (``sq_gemm_split``); without it only whole
    tiles are scheduled."""
    _require_cuda(codes, "codes")
    m, k = codes.shape
    n = packed.shape[0]
    group = w_scales.dtype == torch.float16
    if out is None:
        out = torch.empty((m, n), device=codes.device, dtype=out_dtype)
    acc = None
    if want_accumulators:
        acc = torch.empty((m, n, k // 128 if group else 1), device=codes.device, dtype=torch.int32)
    lib = _lib.load_library()
    layout = int(codes_layout) | (_lib.CODES_INT4_RANGE if int4_range else 0)
    with torch.cuda.device(codes.device):
        if check_kernel or not split:
            fn = lib.sq_gemm_check if check_kernel else lib.sq_gemm
            status = fn(codes.data_ptr(), layout, packed.data_ptr(), w_scales.data_ptr(),
                        _wscale_mode(packed, w_scales), row_scales.data_ptr(), _ptr(bias),
                        out.data_ptr(), _DTYPES[out_dtype], m, n, k, _ptr(acc), _stream())
        else:
            scratch = torch.empty((max(lib.sq_split_workspace_bytes(m), 16),), device=codes.device, dtype=torch.uint8)
            status = lib.sq_gemm_split(codes.data_ptr(), layout, packed.data_ptr(), w_scales.data_ptr(),
                                       _wscale_mode(packed, w_scales), row_scales.data_ptr(), _ptr(bias),
                                       out.data_ptr(), _DTYPES[out_dtype], m, n, k, _ptr(acc),
                                       scratch.data_ptr(), scratch.numel(), _stream())
    _lib.check(status, "sq_gemm_check" if check_kernel else "sq_gemm")
    return (out, acc) if want_accumulators else out


def gemm_scatter(codes: torch.Tensor, packed: torch.Tensor, w_scales: torch.Tensor, row_scales: torch.Tensor, bias,
                 out_pointers, out_ld: int, out_col0: int, *, out_dtype: torch.dtype, int4_range: bool = False):
    """Channel-split GEMM (``sq_gemm_scatter``): this GPU's [M, N] block is stored into columns
    ``[out_col0, out_col0 + N)`` of the row-major [M, out_ld] matrices at ``out_pointers`` - raw device addresses,
    the first one local, the others the same matrix on the other GPUs of the split (peer pointers)."""
    import ctypes
    _require_cuda(codes, "codes")
    m, k = codes.shape
    n = packed.shape[0]
    pointers = (ctypes.c_void_p * len(out_pointers))(*[int(ptr) for ptr in out_pointers])
    layout = int(_lib.CODES_EVEN_ODD) | (_lib.CODES_INT4_RANGE if int4_range else 0)
    with torch.cuda.device(codes.device):
        status = _lib.load_library().sq_gemm_scatter(
            codes.data_ptr(), layout, packed.data_ptr(), w_scales.data_ptr(), _wscale_mode(packed, w_scales),
            row_scales.data_ptr(), _ptr(bias), ctypes.cast(pointers, ctypes.c_void_p), len(out_pointers), int(out_ld),
            int(out_col0), _DTYPES[out_dtype], m, n, k, _stream())
    _lib.check(status, "sq_gemm_scatter")


def _rows_view(t: torch.Tensor, width: int, name: str):
    """(data pointer, row stride in elements, rows) of a tensor whose last axis is contiguous and whose leading
    axes collapse to evenly strided rows - e.g. the strided slice ``modulation[:, 0]`` of a [groups, 6, width] tensor."""
    if t.shape[-1] != width or t.stride(-1) != 1:
        raise ValueError(f"{name} must have a contiguous last axis of {width} elements.")
    flat = t.reshape(-1, width) if t.is_contiguous() else t
    if flat.ndim != 2:
        raise ValueError(f"{name} must be viewable as evenly strided rows.")
    return flat.data_ptr(), (flat.stride(0) if flat.shape[0] > 1 else width), flat.shape[0]


def linear(x: torch.Tensor, packed: torch.Tensor, w_scales: torch.Tensor, bias, *, abits: int, mode: str,
           inverse=None, signs=None, rht_block: int = 128, act_scales=None, gains=None, call: int = 0,
           span: int = 1, streams: int = 1, out: torch.Tensor | None = None,
           workspace: torch.Tensor | None = None, norm: str | None = None, norm_eps: float = 1e-6, norm_weight=None,
           mod_scale=None, mod_shift=None, round_after_norm: bool = False, activation: str | None = None,
           gate=None, residual=None, input_activation: str | None = None, mix=None,
           call_index: torch.Tensor | None = None) -> torch.Tensor:
    """One whole quantized linear (pre-pass + GEMM) through ``sq_linear_fused``.  ``out`` and ``workspace``
    (uint8, at least ``sq_workspace_bytes(rows, K)``) may be passed to reuse buffers across calls.

    Optional fused work: ``input_activation="gelu"`` applied to x first (rounded to x's dtype); ``norm`` ("layer" without affine, or "rms" with optional ``norm_weight``) and AdaLN
    modulation ``(1 + mod_scale) * y + mod_shift`` in front of the quantizer (one modulation row per equal
    share of the input rows), optionally rounded to x's dtype (``round_after_norm``); ``activation="gelu"``,
    ``gate`` (one row per equal share of the output rows) and ``residual`` behind the GEMM:
    ``out = residual + gate * act(linear(x))``.

    ``call_index`` (a CUDA int32 tensor of one element) makes static mode read its schedule entry from device
    memory when the kernel runs instead of taking ``call`` on the host: one captured graph then serves every
    denoise call."""
    _require_cuda(x, "x")
    x = x.contiguous()
    k = x.shape[-1]
    rows = x.numel() // k
    n = packed.shape[0]
    lib = _lib.load_library()
    nbytes = lib.sq_workspace_bytes(rows, k)
    if workspace is None:
        # room for the K-split scratch too (the kernel uses it when the tile count does not fill the SMs evenly)
        nbytes += lib.sq_split_workspace_bytes(rows)
        workspace = torch.empty((max(nbytes, 1),), device=x.device, dtype=torch.uint8)
    elif workspace.numel() < nbytes or workspace.dtype != torch.uint8 or not workspace.is_cuda:
        raise RuntimeError("workspace must be a CUDA uint8 tensor of at least sq_workspace_bytes(rows, K) bytes.")
    else:
        nbytes = workspace.numel()
    if out is None:
        out = torch.empty((*x.shape[:-1], n), device=x.device, dtype=x.dtype)
    elif out.shape != (*x.shape[:-1], n) or out.dtype != x.dtype or not out.is_contiguous():
        raise RuntimeError("out must be a contiguous tensor of shape x.shape[:-1] + (N,) in x's dtype.")
    group = w_scales.dtype == torch.float16
    calls = 0 if act_scales is None else act_scales.numel()
    if call_index is not None and (call_index.dtype != torch.int32 or call_index.numel() != 1
                                   or call_index.device != x.device):
        raise ValueError("call_index must be a one-element int32 tensor on the input's device.")
    if mix is not None:
        # composite rotation (order x power of two); a rotated site takes no block fusion (runtime.py:75-78)
        if (norm is not None or mod_scale is not None or gate is not None or residual is not None
                or activation is not None or input_activation is not None):
            raise ValueError("the composite rotation cannot be combined with fused block work.")
        mix = _mix_matrix(mix, x)
        with torch.cuda.device(x.device):
            status = lib.sq_linear_composite(
                x.data_ptr(), _DTYPES[x.dtype], rows, k, n, int(abits),
                _lib.ACT_TOKEN if mode == "token" else _lib.ACT_STATIC,
                _ptr(inverse), _ptr(signs), mix.data_ptr(), int(mix.shape[0]), _ptr(act_scales), _ptr(gains),
                int(calls), int(call), _ptr(call_index), int(span), int(streams), int(x.shape[-2]),
                packed.data_ptr(), w_scales.data_ptr(), _wscale_mode(packed, w_scales),
                _ptr(bias), out.data_ptr(), workspace.data_ptr(), nbytes, _stream())
        _lib.check(status, "sq_linear_composite")
        return out
    norm_kind = {None: _lib.NORM_NONE, "layer": _lib.NORM_LAYER, "rms": _lib.NORM_RMS}[norm]
    mod_ptr = shift_ptr = gate_ptr = None
    mod_span = gate_span = 1
    mod_stride = gate_stride = 0
    if mod_scale is not None:
        mod_ptr, mod_stride, mod_rows = _rows_view(mod_scale, k, "mod_scale")
        shift_ptr, shift_stride, shift_rows = _rows_view(mod_shift, k, "mod_shift")
        if shift_stride != mod_stride or shift_rows != mod_rows or rows % mod_rows:
            raise ValueError("AdaLN scale and shift must share a layout and cover complete input rows.")
        mod_span = rows // mod_rows
    if gate is not None:
        gate_ptr, gate_stride, gate_rows = _rows_view(gate, n, "gate")
        if rows % gate_rows:
            raise ValueError("Gate groups must cover complete output rows.")
        gate_span = rows // gate_rows
    if residual is not None:
        residual = residual.contiguous()
    with torch.cuda.device(x.device):
        status = lib.sq_linear_scheduled(
            x.data_ptr(), _DTYPES[x.dtype], rows, k, n, int(abits),
            _lib.ACT_TOKEN if mode == "token" else _lib.ACT_STATIC,
            _ptr(inverse), _ptr(signs), int(rht_block), _ptr(act_scales), _ptr(gains), int(calls), int(call),
            _ptr(call_index), int(span), int(streams), int(x.shape[-2]),
            packed.data_ptr(), w_scales.data_ptr(), _wscale_mode(packed, w_scales),
            _ptr(bias), _lib.ACT_FN_GELU if input_activation == "gelu" else _lib.ACT_FN_NONE, norm_kind, float(norm_eps), _ptr(norm_weight), mod_ptr, shift_ptr, int(mod_span),
            int(mod_stride), int(bool(round_after_norm)),
            _lib.ACT_FN_NONE, gate_ptr, int(gate_span), int(gate_stride),
            _ptr(residual), out.data_ptr(), workspace.data_ptr(), nbytes, _stream())
    _lib.check(status, "sq_linear_scheduled")
    if activation == "gelu":  # an output activation is not fused into the GEMM (it measured slower there)
        if gate is not None or residual is not None:
            raise ValueError("an output activation cannot be combined with a fused gate or residual.")
        out = torch.nn.functional.gelu(out)
    return out


TIMELINE_ROLES = ("tma_issue", "unpack_start", "unpack_done", "acc_free", "mma_issue", "drain_start",
                  "acc_released", "drain_done", "mma_committed", "drain_top", "acc_loaded", "item_end")


def gemm_timeline(codes, packed, w_scales, row_scales, bias):
    """``gemm`` for the group-scale bf16 case plus the pipeline timeline of thread block 0: returns
    ``(out, stamps)`` with ``stamps`` an int64 [12, 512] tensor of SM clock values (0 = slot not reached);
    rows are named by ``TIMELINE_ROLES``."""
    _require_cuda(codes, "codes")
    m, k = codes.shape
    n = packed.shape[0]
    out = torch.empty((m, n), device=codes.device, dtype=torch.bfloat16)
    stamps = torch.zeros((len(TIMELINE_ROLES), 512), device=codes.device, dtype=torch.int64)
    with torch.cuda.device(codes.device):
        status = _lib.load_library().sq_gemm_timeline(codes.data_ptr(), packed.data_ptr(), w_scales.data_ptr(),
                                                      row_scales.data_ptr(), _ptr(bias), out.data_ptr(), m, n, k,
                                                      stamps.data_ptr(), _stream())
    _lib.check(status, "sq_gemm_timeline")
    return out, stamps


def mma_rate(n_cols: int = 128, iterations: int = 2000) -> float:
    """SM cycles the tensor pipe takes per ``kind::i8`` MMA of M = 128, N = ``n_cols``, K = 32 when one thread
    issues them back to back (``sq_mma_rate``; synchronises)."""
    cycles = torch.zeros(1, device="cuda", dtype=torch.int64)
    status = _lib.load_library().sq_mma_rate(int(n_cols), int(iterations), cycles.data_ptr(), _stream())
    _lib.check(status, "sq_mma_rate")
    torch.cuda.synchronize()
    return cycles.item() / (4.0 * iterations)


def wait_probe(limit_us: int = 1000) -> int:
    """Run ``sq_wait_probe``: a thread block waits ``limit_us`` microseconds for a barrier nobody arrives at and
    gives up.  Returns the nanoseconds it waited (synchronises); ``device_status()`` afterwards reports 9190 once."""
    waited = torch.zeros(1, device="cuda", dtype=torch.int64)
    _lib.check(_lib.load_library().sq_wait_probe(int(limit_us), waited.data_ptr(), _stream()), "sq_wait_probe")
    torch.cuda.synchronize()
    return int(waited.item())


def device_status() -> int:
    """Read and clear the device-side status word (synchronises)."""
    return int(_lib.load_library().sq_device_status())
