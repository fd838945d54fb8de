"""Host-side logic that needs no GPU: call state, stream layouts, the reference-backend module against the
golden outputs of the reference package, live-graph output validation, operator argument checks."""
import importlib

import pytest
import torch

P = "fastwamjoint_quantization_b200."


@pytest.fixture(scope="module")
def mods(pkg):
    names = ("state", "streams", "topology", "checkpoint", "runtime", "rollout_graph", "quant", "rht", "dit")
    return {n: importlib.import_module(P + n) for n in names}


def test_call_state_and_tracker(mods):
    state = mods["state"].DenoiseCallState(3)
    with pytest.raises(RuntimeError, match="not been set"):
        state.require()
    with pytest.raises(IndexError):
        state.set(3)
    with pytest.raises(ValueError):
        mods["state"].DenoiseCallState(0)

    class Model:
        def __init__(self):
            self.seen = []

        def _predict_joint_noise(self, value):
            self.seen.append(state.require())
            return value

    model = Model()
    with mods["state"].FastWAMCallTracker(model, state) as tracker:
        for i in range(5):
            model._predict_joint_noise(i)
        assert model.seen == [0, 1, 2, 0, 1]
        with pytest.raises(RuntimeError):
            tracker.install()
        tracker.reset()
        assert state.index is None and tracker.total_calls == 0
    assert state.index is None
    model._predict_joint_noise(0) if False else None


def test_stream_layouts(mods):
    S, T = mods["streams"], mods["topology"]
    cfg = S.FastWAMStreamConfig()
    video = T.LinearSite(0, "video", 0, "self_attn.q", "v", None, "expert_tokens")
    action = T.LinearSite(1, "action", 0, "ffn.0", "a", None, "expert_tokens")
    context = T.LinearSite(2, "action", 0, "cross_attn.k", "c", None, "context")
    assert S.resolve_stream_layout(video, 294, cfg).token_counts == (98, 98, 98)
    assert S.resolve_stream_layout(action, 32, cfg).names == ("action_chunk_0", "action_chunk_1")
    layout = S.resolve_stream_layout(context, 129, cfg)
    assert layout.names == ("text", "proprio") and layout.token_counts == (128, 1)
    assert [s.start for s in layout.slices()] == [0, 128]
    with pytest.raises(ValueError, match="divisible"):
        S.resolve_stream_layout(video, 100, cfg)
    x = torch.zeros(2, 129, 4)
    gains = S.expand_stream_gains(x, torch.tensor([2.0, 3.0]), layout)
    assert gains.shape == (1, 129, 1) and gains[0, 127, 0] == 2 and gains[0, 128, 0] == 3
    with pytest.raises(ValueError):
        S.expand_stream_gains(x, torch.ones(3), layout)
    assert T.stream_kind_of("cross_attn.v") == "context" and T.stream_kind_of("ffn.2") == "expert_tokens"


def _site(mods, golden, tag, rotated):
    return mods["checkpoint"].QuantizedSite(
        0, "linear", "action", "self_attn.o", ("action_chunk_0", "action_chunk_1"),
        golden[f"mod_{tag}_qweight"], golden[f"mod_{tag}_wscale"], golden[f"mod_{tag}_d"], golden[f"mod_{tag}_gains"],
        golden[f"mod_{tag}_clips"], torch.full((2, 2), 0.5), 0.0, 0.0, (0.0, 0.0), (0.0, 0.0),
        golden[f"mod_{tag}_signs"] if rotated else None, "rht" if rotated else "none")


@pytest.mark.parametrize("tag", ["plain", "rht"])
def test_reference_backend_module_matches_the_reference_package(mods, golden, tag):
    """``WAMQuantLinear(backend="reference")`` of this package against outputs recorded from the reference's
    own module (K = 256, so the reference's rotation is one 256-point block, which is this package's default)."""
    R, St, Sm = mods["runtime"], mods["state"], mods["streams"]
    source = torch.nn.Linear(256, 8, bias=True, dtype=torch.bfloat16)
    with torch.no_grad():
        source.bias.copy_(golden.bf16(f"mod_{tag}_bias"))
    entry = _site(mods, golden, tag, tag == "rht")
    state = St.DenoiseCallState(2)
    x = golden.bf16(f"mod_{tag}_x")
    for abits in (8, 4):
        module = R.WAMQuantLinear(source, entry, state=state, stream_config=Sm.FastWAMStreamConfig(), weight_bits=4,
                                  activation_bits=abits, backend="reference")
        assert module.in_features == 256 and module.out_features == 8
        with pytest.raises(RuntimeError, match="not been set"):
            state.clear()
            module(x)
        for call in (0, 1):
            state.set(call)
            got = module(x)
            want = golden.bf16(f"mod_{tag}_a{abits}_call{call}_out")
            assert torch.equal(got.view(torch.int16), want.view(torch.int16))


@pytest.mark.parametrize("width", [3072, 1024])
def test_rotated_site_takes_the_reference_rotation_for_its_width(mods, golden, width):
    """A rotated site built WITHOUT a rotation matrix or block: the reference backend of this package must equal
    outputs recorded from the reference's own module, which rotates with had12 x H256 at K = 3072 and with the
    full-width transform at K = 1024 (rht.py:27-39).  A block-local default would fail both."""
    R, St, Sm = mods["runtime"], mods["state"], mods["streams"]
    tag = f"wide{width}"
    source = torch.nn.Linear(width, 8, bias=True, dtype=torch.bfloat16)
    with torch.no_grad():
        source.bias.copy_(golden.bf16(f"mod_{tag}_bias"))
    entry = _site(mods, golden, tag, True)
    state = St.DenoiseCallState(2)
    module = R.WAMQuantLinear(source, entry, state=state, stream_config=Sm.FastWAMStreamConfig(), weight_bits=4,
                              activation_bits=4, backend="reference")
    assert module.official_rotation
    x = golden.bf16(f"mod_{tag}_x")
    for call in (0, 1):
        state.set(call)
        want = golden.bf16(f"mod_{tag}_a4_call{call}_out")
        assert torch.equal(module(x).view(torch.int16), want.view(torch.int16))
    # what the native backend hands to the kernels for the same site
    block, matrix = R.resolve_rotation(width, None, None)
    assert block == 0 and matrix.shape == ((12, 12) if width == 3072 else (2, 2))
    assert R.resolve_rotation(256, None, None) == (256, None)
    assert R.resolve_rotation(3072, 128, None) == (128, None)  # explicit opt-in to a block-local rotation
    with pytest.raises(ValueError, match="3072/14336"):
        R.resolve_rotation(1536, None, None)


def test_module_constructor_refusals(mods, golden):
    R, St, Sm = mods["runtime"], mods["state"], mods["streams"]
    source = torch.nn.Linear(256, 8, bias=False, dtype=torch.bfloat16)
    kwargs = dict(state=St.DenoiseCallState(2), stream_config=Sm.FastWAMStreamConfig(), weight_bits=4)
    plain, rotated = _site(mods, golden, "plain", False), _site(mods, golden, "rht", True)
    with pytest.raises(ValueError, match="Unsupported WAM backend"):
        R.WAMQuantLinear(source, plain, activation_bits=4, backend="triton", **kwargs)
    with pytest.raises(ValueError, match="does not match"):
        R.WAMQuantLinear(source, plain, activation_bits=4, backend="cutlass_w4a8", **kwargs)
    with pytest.raises(ValueError, match="Rotated WAM requires"):
        R.WAMQuantLinear(source, rotated, activation_bits=8, backend="cutlass_w4a8", **kwargs)
    with pytest.raises(ValueError, match="block fusion"):
        R.WAMQuantLinear(source, rotated, activation_bits=4, backend="reference", fuse_block=True, **kwargs)
    with pytest.raises(ValueError, match="gamma_gains"):
        R.WAMQuantLinear(source, plain, activation_bits=4, state=St.DenoiseCallState(3),
                         stream_config=Sm.FastWAMStreamConfig(), weight_bits=4)


def test_operator_argument_checks_raise_value_errors(pkg, oracle):
    ops = importlib.import_module(P + "kernels.w4a8.ops")
    wam = importlib.import_module(P + "kernels.w4a4.wam_ops")
    q = torch.randint(-8, 8, (8, 64), dtype=torch.int8)
    assert torch.equal(ops.pack_signed_int4(q), oracle.pack_signed_int4(q))
    with pytest.raises(ValueError):
        ops.pack_signed_int4(q[:, :63])
    with pytest.raises(ValueError, match="-8, 7"):
        ops.pack_signed_int4(torch.full((8, 64), 9, dtype=torch.int8))
    x = torch.zeros(1, 4, 256, dtype=torch.bfloat16)  # a CPU tensor: refused before anything is launched
    packed = torch.zeros(8, 128, dtype=torch.uint8)
    with pytest.raises(ValueError, match="CUDA"):
        ops.symmetric_dynamic_linear(x, packed, torch.ones(8), None, torch.ones(256))
    with pytest.raises(ValueError, match="CUDA"):
        wam.symmetric_scheduled_stream_linear(x, packed, torch.ones(8), None, torch.ones(256), torch.ones(2),
                                              torch.ones(2, 2), (2, 2), 0)
    with pytest.raises(ValueError, match="CUDA"):
        ops.symmetric_scheduled_stream_adaln_linear(x, packed, torch.ones(8), None, torch.ones(256), torch.ones(2),
                                                    torch.ones(2, 2), (2, 2), 0, x[0, :2], x[0, :2], 1e-6)
    assert ops.load_extension.cache_info().currsize == 0  # never loaded on a box without CUDA


def test_live_graph_output_validation(mods):
    G = mods["rollout_graph"]
    glue = G.LiveJointDiTGraph(object(), num_calls=2)
    a = torch.ones(2, 3)
    glue._validate_outputs((a,), (a.clone(),), 0)
    assert glue.validation_records[-1]["passed"] and glue.validation_records[-1]["max_abs"] == 0
    with pytest.raises(AssertionError):
        glue._validate_outputs((a,), (a + 0.1,), 0)
    assert glue.validation_records[-1]["passed"] is False
    with pytest.raises(RuntimeError, match="Nonfinite"):
        glue._validate_outputs((a * float("nan"),), (a,), 0)
    with pytest.raises(RuntimeError, match="layout"):
        glue._validate_outputs((a,), (a.double(),), 0)
    with pytest.raises(RuntimeError, match="count"):
        glue._validate_outputs((a, a), (a,), 0)
    lenient = G.LiveJointDiTGraph(object(), num_calls=2, allow_numerical_mismatch=True)
    lenient._validate_outputs((a,), (a + 0.1,), 1)
    assert lenient.validation_records[-1] == {"step": 1, "output": 0, "max_abs": pytest.approx(0.1, rel=1e-5),
                                              "rmse": pytest.approx(0.1, rel=1e-5), "passed": False}
    with pytest.raises(ValueError):
        G.LiveJointDiTGraph(object(), num_calls=0)
    with pytest.raises(ValueError, match="CUDA"):
        G._signature(torch.ones(1))


def test_token_linear_reference_backend_matches_oracle(mods, oracle):
    D = mods["dit"]
    for abits, rotate in ((8, False), (4, True)):
        w, x = oracle.synthetic_linear(24, 256, 64, seed=3)
        layer = D.TokenQuantLinear(w.bfloat16(), activation_bits=abits, rotate=rotate, module_name="linear",
                                   backend="reference")
        signs = oracle.rht_signs(256, seed=0, module_name="linear") if rotate else None
        wq = oracle.rotate_weight(w.bfloat16(), signs, torch.bfloat16).float() if rotate else w.bfloat16().float()
        qweight, scales = oracle.quantize_weight_group(wq)
        assert torch.equal(layer.weight, oracle.pack_signed_int4(qweight)) and torch.equal(layer.weight_scales, scales)
        want = oracle.token_module_forward(x, qweight, scales, None, abits=abits, signs=signs)
        assert torch.equal(layer(x).view(torch.int16), want.view(torch.int16))


def test_weight_helpers_match_oracle(mods, oracle, golden):
    Q, H = mods["quant"], mods["rht"]
    w = golden["w_in"]
    q, s = Q.quantize_weight_per_channel(w, bits=4)
    assert torch.equal(q, golden["w_q_channel"]) and torch.equal(s, golden["w_s_channel"])
    qg, sg = Q.quantize_weight_group(w)
    qo, so = oracle.quantize_weight_group(w)
    assert torch.equal(qg, qo) and torch.equal(sg, so)
    assert torch.equal(H.rht_signs(256, seed=42, module_name="blocks.0.q"), golden["signs_256_s42_blocks0q"])
    assert torch.equal(H.block_hadamard(golden["had_in"], 128), golden["had128_out"])
    assert torch.equal(H.randomized_block_hadamard_transform(golden["rot_in"], golden["rot_signs"]), golden["rot_rht_out"])
    v, scale = golden["fq_in"], golden["fq_a4_scale"]
    assert torch.equal(Q.symmetric_fake_quant(v, bits=4, scale=scale), golden["fq_a4_out"])


def test_composite_rotation_helper_matches_the_reference(mods, golden):
    """``rht.randomized_composite_hadamard_transform`` with the reference's own sign matrices against the
    reference's "rht" transform at widths 3072 and 14336 (recorded vectors), bit for bit on the CPU."""
    H = mods["rht"]
    assert H.composite_order(3072) == 12 and H.composite_order(14336) == 28 and H.composite_order(4096) is None
    for order, width in ((12, 3072), (28, 14336)):
        signs = H.rht_signs(width, seed=42, module_name="linear")
        matrix = golden[f"mix{order}_matrix"].float()
        got = H.randomized_composite_hadamard_transform(golden[f"mix{order}_in"], signs, matrix)
        assert torch.equal(got, golden[f"mix{order}_out"])
    with pytest.raises(ValueError):
        H.composite_hadamard(torch.zeros(2, 3072), torch.ones(28, 28))
    with pytest.raises(ValueError):
        H.randomized_composite_hadamard_transform(torch.zeros(2, 96), torch.ones(95), torch.ones(12, 12))


def test_call_state_device_mode_defaults(mods):
    """The device-side call index is opt-in: a fresh state is host-indexed and keeps no device tensors."""
    state = mods["state"].DenoiseCallState(4)
    assert state.on_device is False and state._mirrors == {}
    state.set(2)
    assert state.require() == 2
    assert mods["state"].DenoiseCallState(4) == mods["state"].DenoiseCallState(4)
