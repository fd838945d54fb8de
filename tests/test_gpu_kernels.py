"""Parity of the CUDA kernels with the CPU oracle, through the C ABI.

Bars: activation codes and int32 accumulators bit-exact; post-rotation codes may differ
by at most 1 on at most 0.1 % of elements; outputs within 1e-2 relative Frobenius error
(the cross-check kernel, which keeps the oracle's fp32 operation order, must be bit-exact).
"""
import importlib

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def native(pkg):
    return importlib.import_module("fastwamjoint_quantization_b200.native")


@pytest.fixture(autouse=True)
def no_device_timeouts(native):
    yield
    torch.cuda.synchronize()
    assert native.device_status() == 0, "a kernel gave up a bounded wait"


def even_odd(codes: torch.Tensor) -> torch.Tensor:
    """natural -> even-k-first order inside each run of 8"""
    m, k = codes.shape
    runs = codes.reshape(m, k // 8, 8)
    return torch.cat((runs[..., 0::2], runs[..., 1::2]), dim=-1).reshape(m, k)


def rel_fro(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm()).item()


def assert_codes(got, want, rotated):
    if not rotated:
        assert torch.equal(got, want)
        return
    diff = (got.int() - want.int()).abs()
    assert diff.max() <= 1
    assert (diff != 0).float().mean().item() <= 1e-3


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("m,k", [(1, 128), (33, 1024), (50, 3072), (7, 12288), (5, 14336), (3, 96)])
@pytest.mark.parametrize("abits,rotate", [(8, False), (4, False), (4, True), (8, True)])
def test_prepass_token(native, oracle, dtype, m, k, abits, rotate):
    if rotate and k % 128:
        pytest.skip("rotation block must divide K")
    gen = torch.Generator().manual_seed(m * 131 + k)
    x = torch.randn(m, k, generator=gen)
    x[:, torch.randperm(k, generator=gen)[: max(1, k // 100)]] *= 20
    if m > 2:
        x[1] = 0  # all-zero token: scale clamps at 1e-8, codes are 0
    x = x.to(dtype)
    signs = oracle.rht_signs(k, seed=0, module_name="linear") if rotate else None
    inverse = torch.rand(k, generator=gen) + 0.5 if (m % 2) else None
    want_codes, want_scales = oracle.token_codes(x, bits=abits, signs=signs, inverse=inverse)
    dev = lambda t: None if t is None else t.cuda()
    codes, scales = native.prepass(x.cuda(), abits=abits, mode="token", signs=dev(signs), inverse=dev(inverse),
                                   codes_layout=0)
    assert_codes(codes.cpu(), want_codes, rotate)
    assert torch.equal(scales.cpu(), want_scales)
    codes_eo, _ = native.prepass(x.cuda(), abits=abits, mode="token", signs=dev(signs), inverse=dev(inverse),
                                 codes_layout=1)
    assert torch.equal(codes_eo.cpu(), even_odd(codes.cpu()))
    if abits == 4:
        packed, _ = native.prepass(x.cuda(), abits=4, mode="token", signs=dev(signs), inverse=dev(inverse),
                                   codes_layout=0, pack_int4=True)
        assert torch.equal(packed.cpu(), oracle.pack_signed_int4(codes.cpu()))


@pytest.mark.parametrize("block", [8, 16, 32, 64, 128, 256])
def test_prepass_rotation_blocks(native, oracle, block):
    gen = torch.Generator().manual_seed(block)
    x = (torch.randn(9, 1024, generator=gen) * 2).bfloat16()
    signs = oracle.rht_signs(1024, seed=3, module_name="blocks")
    want, scales = oracle.token_codes(x, bits=8, signs=signs, block=block)
    codes, got_scales = native.prepass(x.cuda(), abits=8, mode="token", signs=signs.cuda(), rht_block=block,
                                       codes_layout=0)
    assert_codes(codes.cpu(), want, True)
    assert torch.allclose(got_scales.cpu(), scales, rtol=1e-6, atol=0)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("m,k,counts,batch", [(32, 1024, (16, 16), 1), (294, 3072, (98, 98, 98), 1),
                                              (129, 1024, (128, 1), 2)])
@pytest.mark.parametrize("abits", [8, 4])
def test_prepass_static_schedule(native, oracle, dtype, m, k, counts, batch, abits):
    """Shapes, layouts and schedule of the reference's own tests (tests/test_wam_w4a4.py:17-36)."""
    gen = torch.Generator().manual_seed(m + k)
    x = (torch.randn(batch, m, k, generator=gen) * 0.5).to(dtype)
    inverse = torch.pow(2.0, torch.randint(-1, 2, (k,), generator=gen).float())
    gains = torch.ones(10, len(counts))
    gains[0] = torch.tensor([0.5, 2.0, 1.0][: len(counts)])
    gains[9] = torch.tensor([2.0, 0.5, 1.0][: len(counts)])
    scales = torch.linspace(0.125, 0.25, 10) if abits == 4 else torch.linspace(0.01, 0.03, 10)
    span = counts[0] if len(set(counts)) == 1 else -counts[1]
    for call in (0, 9):
        want, want_rows = oracle.static_codes(x, bits=abits, inverse=inverse, activation_scales=scales, gains=gains,
                                              token_counts=counts, call=call)
        codes, rows = native.prepass(x.cuda(), abits=abits, mode="static", inverse=inverse.cuda(),
                                     act_scale=scales.cuda()[call:], gains=gains.cuda()[call], span=span,
                                     streams=len(counts), codes_layout=0)
        assert torch.equal(codes.cpu().reshape(batch, m, k), want)
        assert torch.equal(rows.cpu(), want_rows.repeat(batch))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("order,k,rows", [(12, 3072, 50), (28, 14336, 9), (12, 96, 5), (12, 1536, 33), (28, 7168, 3)])
@pytest.mark.parametrize("abits,mode", [(4, "token"), (8, "token"), (4, "static")])
def test_prepass_composite_rotation(native, oracle, golden, dtype, order, k, rows, abits, mode):
    """Composite rotation order x power-of-two (rht.py:27-39) in the pre-pass.  The matrix sum runs in a
    different fp32 order than the CPU matmul of the oracle, so a rotated value may land on the other side of a
    rounding boundary: codes differ by at most 1 on at most 0.1 % of the elements, row scales agree to 1e-6."""
    gen = torch.Generator().manual_seed(order * k + rows)
    matrix = golden[f"mix{order}_matrix"].float()
    x = (torch.randn(rows, k, generator=gen) * 2.0).to(dtype)
    signs = oracle.rht_signs(k, seed=3, module_name="site")
    rotated = oracle.composite_rotate(x.float(), signs, matrix).to(dtype)
    if mode == "token":
        want_codes, want_rows = oracle.token_codes(rotated, bits=abits)
        codes, row_scales = native.prepass(x.cuda(), abits=abits, mode="token", signs=signs.cuda(), mix=matrix.cuda(),
                                           codes_layout=0)
    else:
        inverse = torch.pow(2.0, torch.randint(-1, 2, (k,), generator=gen).float())
        scales = torch.tensor([0.25, 0.5])
        gains = torch.tensor([[1.0], [2.0]])
        want_codes, want_rows = oracle.static_codes(rotated.reshape(1, rows, k), bits=abits, inverse=inverse,
                                                    activation_scales=scales, gains=gains, token_counts=(rows,), call=1)
        want_codes = want_codes.reshape(rows, k)
        codes, row_scales = native.prepass(x.cuda(), abits=abits, mode="static", inverse=inverse.cuda(),
                                           signs=signs.cuda(), mix=matrix.cuda(), act_scale=scales.cuda()[1:],
                                           gains=gains.cuda()[1], span=rows, streams=1, codes_layout=0)
    delta = (codes.cpu().int() - want_codes.int()).abs()
    assert int(delta.max()) <= 1
    assert float((delta != 0).float().mean()) <= 1e-3
    torch.testing.assert_close(row_scales.cpu(), want_rows.reshape(-1).float(), rtol=1e-6, atol=0)


def test_composite_rotation_rejections(native, golden):
    matrix = golden["mix12_matrix"].float().cuda()
    x = torch.zeros(4, 3072, device="cuda", dtype=torch.bfloat16)
    signs = torch.ones(3072, device="cuda")
    with pytest.raises(RuntimeError, match="null"):  # a rotation needs its signs
        native.prepass(x, abits=4, mode="token", mix=matrix)
    with pytest.raises(RuntimeError, match="shape"):  # 3072 / 28 is not an integer
        native.prepass(x, abits=4, mode="token", signs=signs, mix=golden["mix28_matrix"].float().cuda())
    with pytest.raises(ValueError, match="square"):
        native.prepass(x, abits=4, mode="token", signs=signs, mix=matrix[:6])


GEMM_SHAPES = [(256, 1024, 1024), (96, 512, 256), (1, 128, 8), (300, 3072, 384), (17, 256, 136), (520, 1024, 128)]


@pytest.mark.parametrize("m,k,n", GEMM_SHAPES)
@pytest.mark.parametrize("abits", [8, 4])
def test_gemm_group_scheme(native, oracle, m, k, n, abits):
    case = oracle.prepare_token_linear(m, k, n, abits=abits, seed=0)
    want = oracle.linear_token(case["x"], case["qweight"], case["weight_scales"], case["bias"], abits=abits,
                               signs=case["signs"])
    packed = oracle.pack_signed_int4(case["qweight"]).cuda()
    wscales = case["weight_scales"].cuda()
    bias = (torch.randn(n, generator=torch.Generator().manual_seed(n)) * 0.01).bfloat16()
    want_out = oracle.epilogue_group(want["acc"], case["weight_scales"], want["row_scales"], bias, torch.bfloat16)
    codes_nat = want["codes"].cuda()
    row_scales = want["row_scales"].cuda()
    for layout, codes in ((0, codes_nat), (1, even_odd(want["codes"]).cuda())):
        ref_out, ref_acc = native.gemm(codes, packed, wscales, row_scales, bias.cuda(), out_dtype=torch.bfloat16,
                                       codes_layout=layout, want_accumulators=True, check_kernel=True)
        assert torch.equal(ref_acc.cpu().long(), want["acc"])
        assert torch.equal(ref_out.cpu().view(torch.int16), want_out.view(torch.int16))
        out, acc = native.gemm(codes, packed, wscales, row_scales, bias.cuda(), out_dtype=torch.bfloat16,
                               codes_layout=layout, want_accumulators=True)
        assert torch.equal(acc.cpu().long(), want["acc"])
        assert rel_fro(out.cpu(), want_out) < 1e-2
        # same numbers up to the fp32 summation order of the drain: within one bf16 step almost everywhere
        assert rel_fro(out.cpu(), want_out) < 3e-3
        plain = native.gemm(codes, packed, wscales, row_scales, bias.cuda(), out_dtype=torch.bfloat16,
                            codes_layout=layout, split=False)
        assert torch.equal(plain, out)
        parts = native.gemm(codes, packed, wscales, row_scales, bias.cuda(), out_dtype=torch.bfloat16,
                            codes_layout=layout, split=True)
        assert rel_fro(parts.cpu(), want_out) < 3e-3  # parts of a split tile add their fp32 sums in part order
        if abits == 4:  # the promise "codes within [-8, 7]" selects the small accumulator offset
            out4, acc4 = native.gemm(codes, packed, wscales, row_scales, bias.cuda(), out_dtype=torch.bfloat16,
                                     codes_layout=layout, want_accumulators=True, int4_range=True)
            assert torch.equal(acc4.cpu().long(), want["acc"])
            assert rel_fro(out4.cpu(), want_out) < 2e-3


@pytest.mark.parametrize("m,k,n", [(2048, 3072, 3072), (1024, 12288, 3072), (1100, 1024, 4096), (200, 3072, 3072),
                                   (16, 3072, 12288), (16, 3072, 3072), (40, 12288, 3072), (294, 14336, 3072)])
@pytest.mark.parametrize("abits", [8, 4])
def test_gemm_group_scheme_many_tiles(native, oracle, m, k, n, abits):
    """Group form at sizes where a persistent thread block walks several tiles (more tiles than SMs: 384 at
    2048 x 3072 x 3072, the benchmark's headline shape), with 96 groups per tile (K = 12288), with a ragged
    last tile, and below one wave of tiles, where the tiles are split along K.  Every int32 accumulator of the
    tensor-core kernel must equal the CUDA-core cross-check kernel's (itself pinned to the CPU oracle above),
    with and without K-split scratch; a sample of rows is also recomputed by the CPU oracle (the reference's
    exact-test bar, tests/test_wam_w4a4.py:32-58: atol = rtol = 0 on integers)."""
    gen = torch.Generator().manual_seed(m + k + n + abits)
    lim = 8 if abits == 4 else 128
    codes = torch.randint(-lim + 1, lim, (m, k), generator=gen, dtype=torch.int8)
    codes[0, :128] = -lim  # the most negative code the range allows, a whole group long
    qweight = torch.randint(-8, 8, (n, k), generator=gen, dtype=torch.int8)
    wscales = (torch.rand(n, k // 128, generator=gen) * 0.01 + 0.001).half()
    row_scales = torch.rand(m, generator=gen) + 0.5
    bias = (torch.randn(n, generator=gen) * 0.01).bfloat16()
    packed = oracle.pack_signed_int4(qweight).cuda()
    dev_codes = even_odd(codes).cuda()
    args = (dev_codes, packed, wscales.cuda(), row_scales.cuda(), bias.cuda())
    check_out, check_acc = native.gemm(*args, out_dtype=torch.bfloat16, want_accumulators=True, check_kernel=True)
    rows = torch.arange(0, m, 37)
    want_acc = torch.einsum("mgk,ngk->mng", codes[rows].view(len(rows), -1, 128).double(),
                            qweight.view(n, -1, 128).double()).long()
    assert torch.equal(check_acc[rows.cuda()].cpu().long(), want_acc)
    want_out = oracle.epilogue_group(want_acc, wscales, row_scales[rows], bias, torch.bfloat16)
    assert torch.equal(check_out[rows.cuda()].cpu().view(torch.int16), want_out.view(torch.int16))
    for split in (False, True):
        for int4_range in ((False, True) if abits == 4 else (False,)):
            out, acc = native.gemm(*args, out_dtype=torch.bfloat16, want_accumulators=True, int4_range=int4_range,
                                   split=split)
            assert torch.equal(acc, check_acc), (split, int4_range)
            # the drain sums the groups in fp32 in its own order: the bar grows with the number of groups
            bar = 2e-3 if k <= 4096 else 4e-3
            assert rel_fro(out[rows.cuda()].cpu(), want_out) < bar
            assert rel_fro(out, check_out) < bar
            plain = native.gemm(*args, out_dtype=torch.bfloat16, int4_range=int4_range, split=split)
            if split:  # parts of a split tile add their fp32 sums in part order: rounding may differ from one pass
                assert rel_fro(plain, check_out) < bar
            else:
                assert torch.equal(plain, out)
            again = native.gemm(*args, out_dtype=torch.bfloat16, int4_range=int4_range, split=split)
            assert torch.equal(again, plain)  # the K-split reduction does not depend on arrival order
            del out, acc
    assert native.device_status() == 0


@pytest.mark.parametrize("abits", [8, 4])
def test_gemm_at_the_largest_benchmark_size_rows_are_independent(native, oracle, abits):
    """M = 32768, K = 3072, N = 12288 (the largest shape of the benchmark sweep; 24 576 tiles, 166 per SM): too large
    to dump every accumulator, so the check uses what does not depend on size - every output row depends on its
    own codes only.  Slices of 128-aligned and of ragged row ranges, run on their own (where accumulators ARE
    checked against the cross-check kernel), must give the same output bits as the same rows of the full run."""
    m, k, n = 32768, 3072, 12288
    gen = torch.Generator(device="cuda").manual_seed(abits)
    lim = 8 if abits == 4 else 128
    codes = torch.randint(-lim + 1, lim, (m, k), generator=gen, device="cuda", dtype=torch.int8)
    qweight = torch.randint(-8, 8, (n, k), generator=torch.Generator().manual_seed(1), dtype=torch.int8)
    packed = oracle.pack_signed_int4(qweight).cuda()
    wscales = (torch.rand(n, k // 128, generator=gen, device="cuda") * 0.01 + 0.001).half()
    row_scales = torch.rand(m, generator=gen, device="cuda") + 0.5
    full = native.gemm(codes, packed, wscales, row_scales, None, out_dtype=torch.bfloat16, int4_range=(abits == 4))
    for lo, hi in ((0, 256), (16383, 16384 + 130), (m - 300, m)):
        rows, scales = codes[lo:hi].clone(), row_scales[lo:hi].clone()  # fresh allocations: aligned like any tensor
        part, acc = native.gemm(rows, packed, wscales, scales, None, out_dtype=torch.bfloat16,
                                int4_range=(abits == 4), want_accumulators=True)
        check_out, check_acc = native.gemm(rows, packed, wscales, scales, None, out_dtype=torch.bfloat16,
                                           want_accumulators=True, check_kernel=True)
        assert torch.equal(acc, check_acc)
        assert torch.equal(full[lo:hi], part)
        assert rel_fro(part, check_out) < 3e-3
        del part, acc, check_out, check_acc
    assert native.device_status() == 0


@pytest.mark.parametrize("group", [True, False])
def test_channel_split_epilogue_writes_its_columns_into_every_matrix(native, oracle, group):
    """sq_gemm_scatter: the [M, N] block of a GPU that holds N of a layer's channels goes into columns
    [col0, col0 + N) of every [M, ld] matrix it is given (here two matrices on one GPU stand in for the peers);
    the values are those of the plain GEMM bit for bit and nothing outside the block is touched."""
    m, k, n, ld, col0 = 300, 1024, 256, 1024, 512
    gen = torch.Generator().manual_seed(11)
    codes = torch.randint(-7, 8, (m, k), generator=gen, dtype=torch.int8)
    qweight = torch.randint(-8, 8, (n, k), generator=gen, dtype=torch.int8)
    wscales = ((torch.rand(n, k // 128, generator=gen) * 0.01 + 0.001).half() if group
               else torch.rand(n, generator=gen) * 0.01 + 0.001)
    row_scales = torch.rand(m, generator=gen) + 0.5
    bias = (torch.randn(n, generator=gen) * 0.01).bfloat16()
    args = (even_odd(codes).cuda(), oracle.pack_signed_int4(qweight).cuda(), wscales.cuda(), row_scales.cuda(), bias.cuda())
    plain = native.gemm(*args, out_dtype=torch.bfloat16, int4_range=True, split=False)
    first = torch.full((m, ld), 7.0, device="cuda", dtype=torch.bfloat16)
    second = torch.full((m, ld), 7.0, device="cuda", dtype=torch.bfloat16)
    native.gemm_scatter(*args, [first.data_ptr(), second.data_ptr()], ld, col0, out_dtype=torch.bfloat16, int4_range=True)
    torch.cuda.synchronize()
    for matrix in (first, second):
        assert torch.equal(matrix[:, col0:col0 + n], plain)
        assert bool((matrix[:, :col0] == 7.0).all()) and bool((matrix[:, col0 + n:] == 7.0).all())
    with pytest.raises(RuntimeError):
        native.gemm_scatter(*args, [first.data_ptr()], ld, ld - n + 8, out_dtype=torch.bfloat16)  # block past the row end
    assert native.device_status() == 0


@pytest.mark.parametrize("m,k,n", [(16, 3072, 3072), (33, 12288, 3072), (64, 1024, 1024), (7, 512, 136),
                                   (294, 14336, 3072), (360, 12288, 3072)])
def test_channel_form_split_along_k_is_exact(native, oracle, m, k, n):
    """Per-channel scales, few tiles: the parts of a tile split along K exchange int32 accumulators, so the output
    is bit for bit what one pass over K gives, whichever part arrives last and however often the scratch is reused."""
    gen = torch.Generator().manual_seed(m + k + n)
    codes = torch.randint(-127, 128, (m, k), generator=gen, dtype=torch.int8)
    qweight = torch.randint(-8, 8, (n, k), generator=gen, dtype=torch.int8)
    wscales = torch.rand(n, generator=gen) * 0.01 + 0.001
    row_scales = torch.rand(m, generator=gen) + 0.5
    bias = (torch.randn(n, generator=gen) * 0.01).bfloat16()
    args = (even_odd(codes).cuda(), oracle.pack_signed_int4(qweight).cuda(), wscales.cuda(), row_scales.cuda(), bias.cuda())
    one_pass = native.gemm(*args, out_dtype=torch.bfloat16, split=False)
    check_out, _ = native.gemm(*args, out_dtype=torch.bfloat16, want_accumulators=True, check_kernel=True)
    assert torch.equal(one_pass, check_out)
    for _ in range(3):
        assert torch.equal(native.gemm(*args, out_dtype=torch.bfloat16, split=True), one_pass)
    assert native.device_status() == 0


@pytest.mark.parametrize("m,k,n", [(1100, 1024, 200), (1190, 2048, 392), (180, 3072, 136), (40000, 1024, 136)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("with_bias", [True, False])
def test_static_two_warp_drain_edges(native, oracle, m, k, n, dtype, with_bias):
    """The form large problems run (K a multiple of 1024: whole chunks of eight group scales; drain warps of 64 token
    columns; a tile's results stored under the next tile's first groups) at its edges: a last token tile that
    leaves one drain warp of a lane quarter with a few columns or with none, channel counts that are no multiple of
    the 128-channel tile, one round per tile (K = 1024) and several, both output types, with and without bias,
    packed and prepacked weights, and more tiles per thread block than the pending results could be mixed up in
    (m = 40000: 313 token tiles x 2 channel tiles on 148 thread blocks).  The output must equal, bit for bit, that of
    the generic kernel (the one that also dumps its accumulators, which are checked against exact integer sums)."""
    gen = torch.Generator().manual_seed(m + k + n)
    codes = torch.randint(-7, 8, (m, k), generator=gen, dtype=torch.int8)
    qweight = torch.randint(-8, 8, (n, k), generator=gen, dtype=torch.int8)
    wscales = (torch.rand(n, k // 128, generator=gen) * 0.01 + 0.001).half().cuda()
    row_scales = (torch.rand(m, generator=gen) + 0.5).cuda()
    bias = (torch.randn(n, generator=gen) * 0.01).to(dtype).cuda() if with_bias else None
    packed = oracle.pack_signed_int4(qweight).cuda()
    dev_codes = even_odd(codes).cuda()
    generic, acc = native.gemm(dev_codes, packed, wscales, row_scales, bias, out_dtype=dtype, want_accumulators=True,
                               split=False)
    rows = torch.arange(0, m, max(1, m // 40))
    want_acc = torch.einsum("mgk,ngk->mng", codes[rows].view(len(rows), -1, 128).double(),
                            qweight.view(n, -1, 128).double()).long()
    assert torch.equal(acc[rows.cuda()].cpu().long(), want_acc)
    del acc
    for int4_range in (False, True):
        static = native.gemm(dev_codes, packed, wscales, row_scales, bias, out_dtype=dtype, int4_range=int4_range,
                             split=False)
        if not int4_range:
            assert torch.equal(static, generic)
        else:  # another offset constant: the fp32 sums may round differently
            assert rel_fro(static, generic) < 2e-3
        pre = native.gemm(dev_codes, native.prepack_weights(packed), wscales, row_scales, bias, out_dtype=dtype,
                          int4_range=int4_range, split=False)
        assert torch.equal(pre, static)
    assert native.device_status() == 0


@pytest.mark.parametrize("m,k,n", [(300, 3072, 384), (17, 256, 136), (520, 1024, 128), (2048, 1024, 512)])
@pytest.mark.parametrize("group", [True, False])
def test_prepacked_weights_give_the_same_bits(native, oracle, m, k, n, group):
    """sq_prepack_weights turns the packed int4 matrix into the GEMM's operand form (int8 = 16 w, even-odd k);
    the GEMM on it skips the unpack stage and must return exactly what it returns on the packed form."""
    gen = torch.Generator().manual_seed(m + k + n)
    qweight = torch.randint(-8, 8, (n, k), generator=gen, dtype=torch.int8)
    packed = oracle.pack_signed_int4(qweight).cuda()
    tiled = native.prepack_weights(packed)
    assert tiled.dtype == torch.int8 and tiled.shape == (n, k)
    want = (qweight.view(n, k // 8, 4, 2).permute(0, 1, 3, 2).reshape(n, k).int() * 16).to(torch.int8)
    assert torch.equal(tiled.cpu(), want)
    codes = even_odd(torch.randint(-127, 128, (m, k), generator=gen, dtype=torch.int8)).cuda()
    wscales = ((torch.rand(n, k // 128, generator=gen) * 0.01 + 0.001).half() if group
               else torch.rand(n, generator=gen) * 0.01 + 0.001).cuda()
    row_scales = (torch.rand(m, generator=gen) + 0.5).cuda()
    bias = (torch.randn(n, generator=gen) * 0.01).bfloat16().cuda()
    for dtype in (torch.bfloat16, torch.float16):
        b = bias.to(dtype)
        plain = native.gemm(codes, packed, wscales, row_scales, b, out_dtype=dtype)
        pre = native.gemm(codes, tiled, wscales, row_scales, b, out_dtype=dtype)
        assert torch.equal(pre, plain)
    with pytest.raises(RuntimeError, match="enum"):  # natural code order does not match the stored k order
        native.gemm(codes, tiled, wscales, row_scales, None, out_dtype=torch.bfloat16, codes_layout=0)
    with pytest.raises(RuntimeError, match="enum"):
        native.gemm(codes, tiled, wscales, row_scales, None, out_dtype=torch.bfloat16, want_accumulators=True)
    x = (torch.randn(m, k, generator=gen) * 1.5).bfloat16().cuda()
    if group:
        signs = oracle.rht_signs(k, seed=1, module_name="s").cuda()
        assert torch.equal(native.linear(x, tiled, wscales, bias, abits=4, mode="token", signs=signs),
                           native.linear(x, packed, wscales, bias, abits=4, mode="token", signs=signs))


@pytest.mark.parametrize("code,weight,int4_range", [(-128, -8, False), (127, -8, False), (-128, 7, False),
                                                    (127, 7, False), (-8, -8, True), (7, -8, True), (-8, 7, True)])
def test_gemm_group_extreme_sums(native, oracle, code, weight, int4_range):
    """Every product of a 128-K group at the same extreme: the largest sums the integer path can meet."""
    m, k, n = 144, 384, 136
    gen = torch.Generator().manual_seed(7)
    codes = torch.full((m, k), code, dtype=torch.int8)
    qweight = torch.full((n, k), weight, dtype=torch.int8)
    # a few random rows so the case is not rank one
    codes[::5] = torch.randint(-8 if int4_range else -128, 8 if int4_range else 128, codes[::5].shape, generator=gen,
                               dtype=torch.int8)
    qweight[::3] = torch.randint(-8, 8, qweight[::3].shape, generator=gen, dtype=torch.int8)
    wscales = (torch.rand(n, k // 128, generator=gen) * 0.01 + 0.001).half()
    row_scales = torch.rand(m, generator=gen) + 0.5
    want_acc = torch.einsum("mgk,ngk->mng", codes.view(m, -1, 128).long(), qweight.view(n, -1, 128).long())
    want_out = oracle.epilogue_group(want_acc, wscales, row_scales, None, torch.bfloat16)
    packed = oracle.pack_signed_int4(qweight).cuda()
    out, acc = native.gemm(codes.cuda(), packed, wscales.cuda(), row_scales.cuda(), None, out_dtype=torch.bfloat16,
                           codes_layout=0, want_accumulators=True, int4_range=int4_range)
    assert torch.equal(acc.cpu().long(), want_acc)
    assert rel_fro(out.cpu(), want_out) < 2e-3
    plain = native.gemm(codes.cuda(), packed, wscales.cuda(), row_scales.cuda(), None, out_dtype=torch.bfloat16,
                        codes_layout=0, int4_range=int4_range, split=False)
    assert torch.equal(plain, out)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("m,k,n", [(32, 1024, 3072), (32, 3072, 1024), (129, 1024, 3072), (294, 3072, 3072),
                                   (294, 3072, 14336), (294, 14336, 3072)])
def test_gemm_channel_scheme_exact(native, oracle, dtype, m, k, n):
    """The reference's exact W4A4 test (tests/test_wam_w4a4.py:39-58): per-channel scales,
    static schedule, atol = rtol = 0 against the kernel-order oracle."""
    gen = torch.Generator().manual_seed(m + k + n)
    batch = 2 if m == 129 else 1
    x = (torch.randn(batch, m, k, generator=gen) * 0.5).to(dtype)
    qw = torch.randint(-7, 8, (n, k), generator=gen, dtype=torch.int8)
    ws = torch.full((n,), 1 / 512)
    inverse = torch.pow(2.0, torch.randint(-1, 2, (k,), generator=gen).float())
    bias = (torch.randn(n, generator=gen) * 0.01).to(dtype)
    counts = (16, 16) if m == 32 else (128, 1) if m == 129 else (98, 98, 98)
    gains = torch.ones(10, len(counts))
    gains[0] = torch.tensor([0.5, 2.0, 1.0][: len(counts)])
    gains[9] = torch.tensor([2.0, 0.5, 1.0][: len(counts)])
    scales = torch.linspace(0.125, 0.25, 10)
    packed = oracle.pack_signed_int4(qw).cuda()
    span = counts[0] if len(set(counts)) == 1 else -counts[1]
    for call in (0, 9):
        want = oracle.linear_static(x, qw, ws, bias, inverse, scales, gains, counts, call, abits=4)
        out = native.linear(x.cuda(), packed, ws.cuda(), bias.cuda(), abits=4, mode="static", inverse=inverse.cuda(),
                            act_scales=scales.cuda(), gains=gains.cuda(), call=call, span=span, streams=len(counts))
        assert out.shape == (batch, m, n) and out.dtype == dtype
        torch.testing.assert_close(out.cpu(), want["out"], rtol=0, atol=0)
        codes, rows = native.prepass(x.cuda(), abits=4, mode="static", inverse=inverse.cuda(),
                                     act_scale=scales.cuda()[call:], gains=gains.cuda()[call], span=span,
                                     streams=len(counts))
        _, acc = native.gemm(codes, packed, ws.cuda(), rows, bias.cuda(), out_dtype=dtype, want_accumulators=True)
        assert torch.equal(acc.cpu().long()[..., 0], want["acc"])


def test_linear_graph_capture_and_replay_after_mutation(native, oracle):
    """Capture in a CUDA graph, change the input in place, replay: equals a fresh eager run bit for bit
    (tests/test_w4a8.py:32-37)."""
    case = oracle.prepare_token_linear(294, 3072, 3072, abits=8, seed=1)
    x = case["x"].cuda()
    packed = oracle.pack_signed_int4(case["qweight"]).cuda()
    ws = case["weight_scales"].cuda()
    run = lambda: native.linear(x, packed, ws, None, abits=8, mode="token")
    eager = run()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        captured = run()
    graph.replay()
    assert torch.equal(captured, eager)
    x.mul_(0.7)
    graph.replay()
    assert torch.equal(captured, run())


def test_empty_and_ragged_token_counts(native, oracle):
    """Edges of the token axis: no rows at all (nothing is launched, an empty result comes back), one row, and
    counts that leave a partial 16-row MMA column block and a partial tile (129 = 128 + 1, 145 = 128 + 16 + 1),
    on both weight forms; rows past M must not be written."""
    k, n = 512, 264  # N = 2 full channel tiles + 8 channels
    case = oracle.prepare_token_linear(160, k, n, abits=8, seed=4)
    packed = oracle.pack_signed_int4(case["qweight"]).cuda()
    tiled = native.prepack_weights(packed)
    scales, bias = case["weight_scales"].cuda(), case["bias"].cuda()
    empty = native.linear(case["x"][:0].cuda(), packed, scales, bias, abits=8, mode="token")
    assert empty.shape == (0, n) and native.device_status() == 0
    codes, rows = native.prepass(case["x"][:0].cuda(), abits=8, mode="token")
    assert codes.shape == (0, k) and rows.shape == (0,)
    for m in (1, 15, 17, 129, 145, 160):
        x = case["x"][:m]
        want = oracle.linear_token(x, case["qweight"], case["weight_scales"], case["bias"], abits=8,
                                   signs=None, want_accumulators=False)["out"]
        for weight in (packed, tiled):
            guard = torch.full((m + 3, n), 7.0, device="cuda", dtype=torch.bfloat16)
            out = native.linear(x.cuda(), weight, scales, bias, abits=8, mode="token", out=guard[:m])
            assert rel_fro(out.cpu(), want) < 2e-3
            assert torch.all(guard[m:] == 7.0)  # nothing written past the last row
    assert native.device_status() == 0


def test_mma_rate_probe(native):
    """The tensor-pipe probe runs, finishes (bounded wait, status 0) and reports a plausible time per MMA:
    at least the 32 cycles a K = 32 step of 128 x 64 would take at twice the nominal rate, at most 1000."""
    for n_cols in (64, 128, 256):
        cycles = native.mma_rate(n_cols, 500)
        assert 32.0 <= cycles <= 1000.0, (n_cols, cycles)
    assert native.device_status() == 0
    with pytest.raises(RuntimeError, match="enum"):
        native.mma_rate(96, 10)


def test_a_wait_that_runs_out_becomes_a_status(native, oracle):
    """The bounded wait of the pipeline roles, made to run out on purpose in the allowed way: a barrier nobody
    arrives at, a limit of one millisecond.  The kernel returns, the status word names the wait, tensor memory
    was released (a full 512-column GEMM right after gets its allocation and is exact), and the status is clear
    again."""
    assert native.device_status() == 0
    waited = native.wait_probe(1000)
    assert 1_000_000 <= waited < 50_000_000, waited
    status = native.device_status()
    lib = importlib.import_module("fastwamjoint_quantization_b200._lib")
    assert status == 9190 and "wait probe" in lib.status_string(status)
    assert native.device_status() == 0  # reading clears it
    case = oracle.prepare_token_linear(300, 1024, 384, abits=8, seed=5)
    want = oracle.linear_token(case["x"], case["qweight"], case["weight_scales"], case["bias"], abits=8, signs=None)
    packed = oracle.pack_signed_int4(case["qweight"]).cuda()
    _, acc = native.gemm(even_odd(want["codes"]).cuda(), packed, case["weight_scales"].cuda(),
                         want["row_scales"].cuda(), None, out_dtype=torch.bfloat16, want_accumulators=True)
    assert torch.equal(acc.cpu().long(), want["acc"])
    assert native.device_status() == 0
    with pytest.raises(RuntimeError, match="shape"):
        native.wait_probe(0)


def test_rejected_calls_raise(native, oracle):
    case = oracle.prepare_token_linear(8, 256, 16, abits=8, seed=0)
    packed = oracle.pack_signed_int4(case["qweight"]).cuda()
    with pytest.raises(RuntimeError, match="index"):
        native.linear(case["x"].cuda(), packed, torch.ones(16).cuda(), None, abits=8, mode="static",
                      inverse=torch.ones(256).cuda(), act_scales=torch.ones(2).cuda(), gains=torch.ones(2, 2).cuda(),
                      call=2, span=4, streams=2)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        native.prepass(case["x"], abits=8, mode="token")
