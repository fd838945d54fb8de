"""The CPU oracle against outputs recorded from the reference package itself
(``tests/golden/make_golden.py``).  Bit-exact unless a tolerance is written."""
import pytest
import torch


def test_signs(oracle, golden):
    assert torch.equal(oracle.rht_signs(64, seed=0, module_name="linear"), golden["signs_64_s0_linear"])
    assert torch.equal(oracle.rht_signs(256, seed=42, module_name="blocks.0.q"), golden["signs_256_s42_blocks0q"])
    assert torch.equal(oracle.rht_signs(3072, seed=0, module_name="linear")[:64], golden["signs_3072_s0_linear_head"])


def test_block_hadamard_128(oracle, golden):
    assert torch.equal(oracle.block_hadamard(golden["had_in"], 128), golden["had128_out"])


def test_rotation_wrappers(oracle, golden):
    x, signs = golden["rot_in"], golden["rot_signs"]
    # K = 256: the reference's "rht" and "block" modes are both one 256-point block
    assert torch.equal(oracle.rht_rotate(x, signs, 256), golden["rot_rht_out"])
    assert torch.equal(oracle.rht_rotate(x, signs, 256), golden["rot_block_out"])
    xb = golden.bf16("rot_bf16_in")
    got = oracle.rht_rotate(xb.float(), signs, 256).to(torch.bfloat16)
    assert torch.equal(got.view(torch.int16), golden.bf16("rot_bf16_out").view(torch.int16))


def test_composite_rotation_3072_and_14336(oracle, golden):
    """had12 x H256 and had28 x H512 (rht.py:27-39).  The restatement follows the reference operation by
    operation on the CPU, so it is bit-exact there; the sign matrices are the reference's own."""
    for order, width in ((12, 3072), (28, 14336)):
        matrix = golden[f"mix{order}_matrix"]
        assert matrix.shape == (order, order) and set(matrix.flatten().tolist()) == {-1, 1}
        assert torch.equal(matrix.long() @ matrix.long().T, order * torch.eye(order, dtype=torch.long))
        signs = oracle.rht_signs(width, seed=42, module_name="linear")
        x = golden[f"mix{order}_in"]
        assert torch.equal(oracle.composite_rotate(x, signs, matrix), golden[f"mix{order}_out"])
        got = oracle.composite_rotate(x.bfloat16().float(), signs, matrix).to(torch.bfloat16)
        assert torch.equal(got.view(torch.int16), golden.bf16(f"mix{order}_out").view(torch.int16))


def test_fake_quant_and_token_codes(oracle, golden):
    v = golden["fq_in"]
    for bits in (8, 4):
        scale = golden[f"fq_a{bits}_scale"]
        assert torch.equal(oracle.symmetric_fake_quant(v, bits=bits, scale=scale), golden[f"fq_a{bits}_out"])
        # token_codes reproduces the same numbers as codes * scale
        codes, row_scales = oracle.token_codes(v.bfloat16().float(), bits=bits)
        again = oracle.symmetric_fake_quant(v.bfloat16().float(), bits=bits,
                                            scale=v.bfloat16().float().abs().amax(-1, keepdim=True) / (2 ** (bits - 1) - 1))
        assert torch.equal(codes.float() * (v.bfloat16().float().abs().amax(-1, keepdim=True) / (2 ** (bits - 1) - 1)), again)
        assert codes.abs().max() <= 2 ** (bits - 1) - 1
        assert torch.all(row_scales >= 1e-8)
    assert torch.equal(oracle.symmetric_fake_quant(golden["fq_ties_in"], bits=4, scale=torch.ones(1, 1)),
                       golden["fq_ties_out"])


def test_weight_quantizers_and_packing(oracle, golden):
    w = golden["w_in"]
    q, s = oracle.quantize_weight_per_channel(w)
    assert torch.equal(q, golden["w_q_channel"]) and torch.equal(s, golden["w_s_channel"])
    # group form: same arithmetic on [N*K/128, 128]; with the scale rounded to fp16 the codes
    # may move, so pin the un-rounded arithmetic and check the fp16 variant is self-consistent
    qg, sg = oracle.quantize_weight_per_channel(w.reshape(32, 128))
    assert torch.equal(qg.reshape(16, 256), golden["w_q_group_fp32scale"])
    assert torch.equal(sg.reshape(16, 2), golden["w_s_group_fp32scale"])
    q16, s16 = oracle.quantize_weight_group(w)
    assert s16.dtype == torch.float16 and s16.shape == (16, 2)
    assert torch.equal(s16, golden["w_s_group_fp32scale"].half())
    expect = (w.reshape(32, 128) / s16.float().reshape(32, 1)).round().clamp(-7, 7).to(torch.int8)
    assert torch.equal(q16, expect.reshape(16, 256))
    packed = oracle.pack_signed_int4(golden["pack_in"])
    assert torch.equal(packed, golden["pack_out"])
    assert torch.equal(oracle.unpack_signed_int4(packed), golden["pack_in"])


def test_reference_module_forward(oracle, golden):
    for tag in ("plain", "rht"):
        x = golden.bf16(f"mod_{tag}_x")
        signs = golden[f"mod_{tag}_signs"] if tag == "rht" else None
        for abits in (8, 4):
            for call in (0, 1):
                got = oracle.reference_module_forward(
                    x, golden[f"mod_{tag}_qweight"], golden[f"mod_{tag}_wscale"], golden.bf16(f"mod_{tag}_bias"),
                    golden[f"mod_{tag}_d"], golden[f"mod_{tag}_clips"], golden[f"mod_{tag}_gains"], (16, 16), call,
                    abits=abits, signs=signs)
                want = golden.bf16(f"mod_{tag}_a{abits}_call{call}_out")
                assert torch.equal(got.view(torch.int16), want.view(torch.int16)), (tag, abits, call)


def test_kernel_order_oracle_matches_module_on_power_of_two_values(oracle):
    """The multiplying kernel order and the dividing CPU module agree exactly when D,
    gains and scales are powers of two (the condition of the reference's own exact
    test, tests/test_wam_w4a4.py:115-145)."""
    gen = torch.Generator().manual_seed(3)
    qweight = torch.randint(-7, 8, (8, 256), generator=gen, dtype=torch.int8)
    wscale = torch.full((8,), 1 / 64)
    dvec = torch.ones(256) * 2
    gains = torch.tensor([[0.5, 2.0], [2.0, 0.5]])
    clips = torch.tensor([1.75, 3.5])
    x = torch.randn(2, 32, 256, generator=gen).bfloat16()
    for call in (0, 1):
        module = oracle.reference_module_forward(x, qweight, wscale, None, dvec, clips, gains, (16, 16), call, abits=4)
        kernel = oracle.linear_static(x, qweight, wscale, None, dvec.reciprocal(), clips / 7, gains, (16, 16), call,
                                      abits=4)
        assert torch.equal(module.float(), kernel["out"].float())


def test_accumulators_are_exact_integers(oracle):
    gen = torch.Generator().manual_seed(11)
    codes = torch.randint(-127, 128, (9, 256), generator=gen, dtype=torch.int8)
    qweight = torch.randint(-8, 8, (24, 256), generator=gen, dtype=torch.int8)
    acc = oracle.group_accumulators(codes, qweight, 128)
    want = torch.einsum("mgk,ngk->mng", codes.reshape(9, 2, 128).long(), qweight.reshape(24, 2, 128).long())
    assert torch.equal(acc, want)
    assert torch.equal(oracle.group_accumulators(codes, qweight, None)[..., 0], want.sum(-1))


def test_official_rotation_is_selected_by_the_width(oracle, golden):
    """``official_rotate`` against the reference's ``rht_transform(..., "rht")``: matrices rebuilt from the masks,
    full-width transform at 256 and 1024, had12 x H256 at 3072, had28 x H512 at 14336."""
    for order in (12, 28):
        assert torch.equal(oracle.official_matrix(order), golden[f"mix{order}_matrix"].float())
    assert torch.equal(oracle.official_rotate(golden["rot_in"], golden["rot_signs"]), golden["rot_rht_out"])
    for order, width in ((12, 3072), (28, 14336)):
        signs = oracle.rht_signs(width, seed=42, module_name="linear")
        assert torch.equal(oracle.official_rotate(golden[f"mix{order}_in"], signs), golden[f"mix{order}_out"])
    for width in (3072, 1024):
        x = golden.bf16(f"mod_wide{width}_x")
        got = oracle.official_rotate(x.float(), golden[f"mod_wide{width}_signs"]).bfloat16()
        assert torch.equal(got.view(torch.int16), golden.bf16(f"rot_wide{width}_out").view(torch.int16))
    with pytest.raises(ValueError, match="3072/14336"):
        oracle.official_rotate(torch.zeros(1, 1536), torch.ones(1536))
