"""The shared library loads and exports every symbol ``include/sq_b200.h`` declares
(no compute calls: this runs without a GPU), and host-side argument checks reject
bad calls before any launch."""
import ctypes
import importlib
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


@pytest.fixture(scope="module")
def lib(pkg):
    import __graft_entry__ as entry
    entry.build()
    return importlib.import_module("fastwamjoint_quantization_b200._lib")


def test_header_symbols_are_exported(lib):
    header = (ROOT / "include" / "sq_b200.h").read_text()
    declared = set(re.findall(r"^(?:int|size_t|const char\*)\s+(sq_\w+)\s*\(", header, flags=re.M))
    assert declared, "no declarations parsed from the header"
    handle = lib.load_library()
    for name in declared:
        assert hasattr(handle, name), f"{name} is declared but not exported"
    assert declared == set(lib.EXPORTED)


def test_status_strings_and_version(lib):
    handle = lib.load_library()
    assert handle.sq_version().decode().startswith("sq_b200")
    assert lib.status_string(0) == "ok"
    assert "index" in lib.status_string(lib.ERR_INDEX)
    assert "workspace" in lib.status_string(lib.ERR_WORKSPACE)


def test_workspace_bytes(lib):
    handle = lib.load_library()
    assert handle.sq_workspace_bytes(0, 1024) == 0
    assert handle.sq_workspace_bytes(3, 1024) == 3 * 1024 + 256
    assert handle.sq_workspace_bytes(2048, 3072) == 2048 * 3072 + 2048 * 4


def test_argument_errors_need_no_gpu(lib):
    handle = lib.load_library()
    fake = ctypes.c_void_p(4096)  # never dereferenced: rejected before any launch
    # null pointers
    assert handle.sq_prepass(None, 0, 4, 256, 8, 1, None, None, 0, None, None, 1, 1, 4, 0, 0, fake, fake, None) == lib.ERR_NULL
    # K not a multiple of 8
    assert handle.sq_prepass(fake, 0, 4, 250, 8, 1, None, None, 0, None, None, 1, 1, 4, 0, 0, fake, fake, None) == lib.ERR_SHAPE
    # bad bit width
    assert handle.sq_prepass(fake, 0, 4, 256, 5, 1, None, None, 0, None, None, 1, 1, 4, 0, 0, fake, fake, None) == lib.ERR_ENUM
    # rotation block not a power of two
    assert handle.sq_prepass(fake, 0, 4, 384, 4, 1, None, fake, 96, None, None, 1, 1, 4, 0, 0, fake, fake, None) == lib.ERR_SHAPE
    # GEMM: group scales need K % 128 == 0; N % 8 != 0; out-of-range schedule index in sq_linear
    assert handle.sq_gemm(fake, 1, fake, fake, 1, fake, None, fake, 0, 4, 8, 160, None, None) == lib.ERR_SHAPE
    assert handle.sq_gemm(fake, 1, fake, fake, 0, fake, None, fake, 0, 4, 7, 256, None, None) == lib.ERR_SHAPE
    assert handle.sq_linear(fake, 0, 4, 256, 8, 4, 0, fake, None, 0, fake, fake, 10, 10, 2, 2, 4,
                            fake, fake, 0, None, fake, fake, 1 << 20, None) == lib.ERR_INDEX
    assert handle.sq_linear(fake, 0, 4, 256, 8, 4, 0, fake, None, 0, fake, fake, 10, 0, 2, 2, 4,
                            fake, fake, 0, None, fake, fake, 16, None) == lib.ERR_WORKSPACE


def test_misaligned_pointers_are_rejected_on_the_host(lib):
    """Every pointer a kernel reads or writes as a 16-byte vector is checked before anything is launched: a
    pointer that is off by 4 bytes comes back as SQ_ERR_SHAPE instead of faulting on the device."""
    handle = lib.load_library()
    ok, off = ctypes.c_void_p(4096), ctypes.c_void_p(4096 + 4)
    prepass = lambda x, inv_d, signs, codes: handle.sq_prepass(x, 0, 4, 256, 8, 1, inv_d, signs, 128, None, None, 1, 1,
                                                               4, 0, 0, codes, ok, None)
    assert prepass(off, None, None, ok) == lib.ERR_SHAPE      # x
    assert prepass(ok, off, None, ok) == lib.ERR_SHAPE        # 1 / D
    assert prepass(ok, None, off, ok) == lib.ERR_SHAPE        # signs
    assert prepass(ok, None, None, off) == lib.ERR_SHAPE      # codes
    gemm = lambda codes, packed, rows, out: handle.sq_gemm(codes, 1, packed, ok, 1, rows, None, out, 0, 4, 8, 256,
                                                           None, None)
    assert gemm(off, ok, ok, ok) == lib.ERR_SHAPE
    assert gemm(ok, off, ok, ok) == lib.ERR_SHAPE
    assert gemm(ok, ok, off, ok) == lib.ERR_SHAPE             # row scales are read four at a time
    assert gemm(ok, ok, ok, off) == lib.ERR_SHAPE
    # the fused entry: modulation rows and the norm weight
    fused = lambda norm_weight, mod: handle.sq_linear_fused(
        ok, 0, 4, 256, 8, 8, 1, None, None, 128, None, None, 0, 0, 1, 1, 4, ok, ok, 1, None,
        0, 2, 1e-6, norm_weight, mod, mod, 1, 256, 0, 0, None, 1, 0, None, ok, ok, 1 << 20, None)
    assert fused(off, None) == lib.ERR_SHAPE
    assert fused(None, off) == lib.ERR_SHAPE
    # K-split scratch of sq_gemm_split
    assert handle.sq_gemm_split(ok, 1, ok, ok, 1, ok, None, ok, 0, 4, 8, 256, None, off, 1 << 20, None) == lib.ERR_SHAPE
    assert handle.sq_split_workspace_bytes(0) == 0
    assert handle.sq_split_workspace_bytes(16) >= 1024 + 2 * 16 * 128 * 4
