"""``sq_linear_noalloc``: the whole linear with scratch owned by the library, for callers that cannot
allocate device memory (a loop that must not stall on cudaMalloc, a host whose pool already owns the
GPU's memory, a plug-in that gets pointers but no allocator).

Collected last on purpose, so a run that stops at the first failure has already run everything else.
Called through the C ABI with raw pointers; compared with ``sq_linear`` (caller-provided scratch) on the
same inputs, bit for bit, on two calls in a row - the second call meets the first call's leftovers in
the shared array."""
import ctypes
import importlib

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call(lib, fn_name, x, packed, scales, out, abits, signs, workspace=None):
    rows, k = x.shape
    n = packed.shape[0]
    group = scales.dtype == torch.float16
    head = [x.data_ptr(), 0, rows, k, n, abits, 1, None, None if signs is None else signs.data_ptr(), 128,
            None, None, 0, 0, 1, 1, rows, packed.data_ptr(), scales.data_ptr(), 1 if group else 0, None, out.data_ptr()]
    stream = torch.cuda.current_stream().cuda_stream
    if workspace is None:
        return getattr(lib, fn_name)(*head, stream)
    return getattr(lib, fn_name)(*head, workspace.data_ptr(), workspace.numel(), stream)


@pytest.mark.parametrize("abits", [8, 4])
def test_no_alloc_entry_matches_sq_linear_twice(pkg, oracle, abits):
    _lib = importlib.import_module("fastwamjoint_quantization_b200._lib")
    lib = _lib.load_library()
    outs = []
    for m, k, n, seed in ((300, 1024, 512, 1), (96, 3072, 256, 2)):  # two calls in a row, different sizes
        case = oracle.prepare_token_linear(m, k, n, abits=abits, seed=seed)
        x = case["x"].cuda()
        packed = oracle.pack_signed_int4(case["qweight"]).cuda()
        scales = case["weight_scales"].cuda()
        signs = None if case["signs"] is None else case["signs"].cuda()
        want = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
        workspace = torch.empty(lib.sq_workspace_bytes(m, k), device="cuda", dtype=torch.uint8)
        assert _call(lib, "sq_linear", x, packed, scales, want, abits, signs, workspace) == 0
        got = torch.full((m, n), float("nan"), device="cuda", dtype=torch.bfloat16)
        # first call on this shape: may look the scratch address up and load kernel images
        assert _call(lib, "sq_linear_noalloc", x, packed, scales, got, abits, signs) == 0
        torch.cuda.synchronize()
        # a warm call must leave the device's free memory untouched: mem_get_info is the driver's own count,
        # so it also sees a cudaMalloc that bypasses torch's allocator
        steady = False
        for _ in range(3):  # the count is device-wide; retry in case something else on the device moved it
            free_before, _ = torch.cuda.mem_get_info()
            got.fill_(float("nan"))
            assert _call(lib, "sq_linear_noalloc", x, packed, scales, got, abits, signs) == 0
            torch.cuda.synchronize()
            free_after, _ = torch.cuda.mem_get_info()
            steady = steady or free_after == free_before
        assert steady
        assert torch.equal(got.view(torch.int16), want.view(torch.int16))  # tolerance: none, the paths are the same kernels
        ref = oracle.linear_token(case["x"], case["qweight"], case["weight_scales"], case["bias"], abits=abits,
                                  signs=case["signs"], want_accumulators=False)["out"]
        err = ((got.cpu().float() - ref.float()).norm() / ref.float().norm()).item()
        assert err < 1e-2
        outs.append(got)
    assert lib.sq_device_status() == 0


def test_no_alloc_entry_rejects_oversized_calls(pkg):
    _lib = importlib.import_module("fastwamjoint_quantization_b200._lib")
    lib = _lib.load_library()
    fake = ctypes.c_void_p(4096)  # never dereferenced: the size check comes first
    status = lib.sq_linear_noalloc(fake, 0, 4096, 3072, 3072, 8, 1, None, None, 128, None, None, 0, 0, 1, 1, 4096,
                                   fake, fake, 1, None, fake, None)
    assert status == _lib.ERR_SCRATCH_LIMIT
    assert "scratch" in _lib.status_string(status)
