"""ctypes binding of ``libsq_b200.so`` (C ABI declared in ``include/sq_b200.h``).

There is no fallback: if the library has not been built, or no CUDA device is
present when a kernel is requested, the call raises.
"""
from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_float, c_int, c_int64, c_size_t, c_void_p
from functools import lru_cache
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "lib" / "libsq_b200.so"

# status codes of include/sq_b200.h
OK, ERR_NULL, ERR_SHAPE, ERR_ENUM, ERR_INDEX, ERR_DRIVER, ERR_WORKSPACE, ERR_DEVICE_WAIT = 0, -1, -2, -3, -4, -5, -6, -7
ERR_SCRATCH_LIMIT = -8
NOALLOC_SCRATCH_BYTES = 8 * 1024 * 1024 + 65536
BF16, FP16 = 0, 1
ACT_STATIC, ACT_TOKEN = 0, 1
CODES_NATURAL, CODES_EVEN_ODD = 0, 1
WEIGHTS_PREPACKED = 4  # OR-ed onto the weight-scale mode: weights are int8 [N, K] from sq_prepack_weights
CODES_INT4_RANGE = 2  # OR-ed onto the layout for sq_gemm: every code lies in [-8, 7]
WSCALE_CHANNEL_F32, WSCALE_GROUP_F16 = 0, 1
NORM_NONE, NORM_LAYER, NORM_RMS = 0, 1, 2
ACT_FN_NONE, ACT_FN_GELU = 0, 1

_SIGNATURES = {
    "sq_prepass": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int, c_int, c_void_p, c_void_p, c_int,
                           c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "sq_gemm": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
                        c_int64, c_int64, c_int64, c_void_p, c_void_p]),
    "sq_gemm_split": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
                              c_int64, c_int64, c_int64, c_void_p, c_void_p, c_size_t, c_void_p]),
    "sq_split_workspace_bytes": (c_size_t, [c_int64]),
    "sq_gemm_scatter": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int64,
                                c_int64, c_int, c_int64, c_int64, c_int64, c_void_p]),
    "sq_gemm_check": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
                              c_int64, c_int64, c_int64, c_void_p, c_void_p]),
    "sq_gemm_timeline": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                                 c_void_p, c_void_p]),
    "sq_prepack_weights": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_void_p]),
    "sq_mma_rate": (c_int, [c_int, c_int, c_void_p, c_void_p]),
    "sq_workspace_bytes": (c_size_t, [c_int64, c_int64]),
    "sq_linear": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_int, c_int, c_void_p, c_void_p, c_int,
                          c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64,
                          c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p]),
    "sq_linear_fused": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_int, c_int, c_void_p, c_void_p, c_int,
                                c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64,
                                c_void_p, c_void_p, c_int, c_void_p,
                                c_int, c_int, c_float, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int,
                                c_int, c_void_p, c_int64, c_int64, c_void_p,
                                c_void_p, c_void_p, c_size_t, c_void_p]),
    "sq_linear_scheduled": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_int, c_int, c_void_p, c_void_p, c_int,
                                    c_void_p, c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_int64,
                                    c_void_p, c_void_p, c_int, c_void_p,
                                    c_int, c_int, c_float, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int,
                                    c_int, c_void_p, c_int64, c_int64, c_void_p,
                                    c_void_p, c_void_p, c_size_t, c_void_p]),
    "sq_prepass_composite": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                     c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int, c_int, c_void_p, c_void_p,
                                     c_void_p]),
    "sq_linear_composite": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_int, c_int, c_void_p, c_void_p,
                                    c_void_p, c_int, c_void_p, c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_int64,
                                    c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p]),
    "sq_linear_noalloc": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_int, c_int, c_void_p, c_void_p, c_int,
                                  c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64,
                                  c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p]),
    "sq_wait_probe": (c_int, [c_int64, c_void_p, c_void_p]),
    "sq_device_status": (c_int, []),
    "sq_status_string": (c_char_p, [c_int]),
    "sq_version": (c_char_p, []),
}

EXPORTED = tuple(_SIGNATURES)


@lru_cache(maxsize=1)
def load_library() -> ctypes.CDLL:
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python {LIB_PATH.parents[1] / 'build.py'}` "
            "(needs nvcc). There is no fallback path.")
    lib = ctypes.CDLL(str(LIB_PATH))
    for name, (restype, argtypes) in _SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = restype
        fn.argtypes = argtypes
    return lib


def status_string(status: int) -> str:
    return load_library().sq_status_string(int(status)).decode()


def check(status: int, what: str) -> None:
    """Turn a non-zero status into the exception type the reference raises at the
    same place: argument errors found by its C++ checks are RuntimeError
    (TORCH_CHECK, kernels/w4a8/csrc/w4a8.cu:1079-1115)."""
    if status != OK:
        raise RuntimeError(f"{what}: {status_string(status)} (status {status})")
