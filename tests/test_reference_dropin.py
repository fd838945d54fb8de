"""Drop-in proof: the REFERENCE's own ``WAMQuantLinear`` and ``LiveJointDiTGraph`` (a copy of its pure-Python
package under ``oracle/_ref``, made by ``oracle/make_ref.py``) running on THIS library's operator modules.

Only ``fastwam_steerquant.kernels.w4a8.ops`` and ``fastwam_steerquant.kernels.w4a4.wam_ops`` are swapped - the two
modules the reference binds its CUDA extensions through (runtime.py:27-31, 82-86).  Everything else - module,
call state, stream layouts, graph glue - is the reference's code.  Cases: its exact native == reference-backend
test (tests/test_wam_w4a4.py:115-145), its rotated shapes (tests/test_rht.py:101-150), its live-graph test
(tests/test_rollout_graph.py:62-87).  Skipped when the copy is absent."""
import importlib
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
REF_ROOT = Path(__file__).resolve().parents[1] / "oracle" / "_ref"


@pytest.fixture(scope="module")
def ref(pkg):
    if not (REF_ROOT / "fastwam_steerquant" / "runtime.py").exists():
        pytest.skip("oracle/_ref is absent (python oracle/make_ref.py makes it where the reference checkout is)")
    ours8 = importlib.import_module("fastwamjoint_quantization_b200.kernels.w4a8.ops")
    ours4 = importlib.import_module("fastwamjoint_quantization_b200.kernels.w4a4.wam_ops")
    saved = {name: module for name, module in sys.modules.items() if name.split(".")[0] == "fastwam_steerquant"}
    for name in saved:
        del sys.modules[name]
    sys.path.insert(0, str(REF_ROOT))
    # the swap: the reference imports these two names and gets this library's operators
    sys.modules["fastwam_steerquant.kernels.w4a8.ops"] = ours8
    sys.modules["fastwam_steerquant.kernels.w4a4.wam_ops"] = ours4
    try:
        import fastwam_steerquant  # noqa: F401
        names = ("runtime", "checkpoint", "state", "streams", "rht", "rollout_graph")
        modules = {name: importlib.import_module("fastwam_steerquant." + name) for name in names}
        assert Path(modules["runtime"].__file__).is_relative_to(REF_ROOT)
        assert importlib.import_module("fastwam_steerquant.kernels.w4a4").wam_ops is ours4
        yield modules
    finally:
        sys.path.remove(str(REF_ROOT))
        for name in [n for n in sys.modules if n.split(".")[0] == "fastwam_steerquant"]:
            del sys.modules[name]
        sys.modules.update(saved)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("abits", [4, 8])
def test_reference_module_native_backend_equals_its_reference_backend(ref, monkeypatch, dtype, abits):
    monkeypatch.setattr(torch.backends.cuda.matmul, "allow_bf16_reduced_precision_reduction", False)
    R, C, S, St = ref["runtime"], ref["checkpoint"], ref["streams"], ref["state"]
    source = torch.nn.Linear(256, 8, bias=False, device="cuda", dtype=dtype)
    entry = C.QuantizedSite(
        0, "linear", "action", "self_attn.o", ("action_chunk_0", "action_chunk_1"),
        torch.randint(-7, 8, (8, 256), dtype=torch.int8), torch.full((8, 1), 1 / 64), torch.ones(256) * 2,
        torch.tensor([[0.5, 2.0], [2.0, 0.5]]), torch.tensor([1.75, 3.5]), torch.full((2, 2), 0.5), 0.0, 0.0,
        (0.0, 0.0), (0.0, 0.0))
    state = St.DenoiseCallState(2)
    kwargs = dict(state=state, stream_config=S.FastWAMStreamConfig(), weight_bits=4, activation_bits=abits)
    native = R.WAMQuantLinear(source, entry, backend=f"cutlass_w4a{abits}", **kwargs)
    reference = R.WAMQuantLinear(source, entry, backend="reference", **kwargs)
    assert type(native).__module__ == "fastwam_steerquant.runtime"
    assert native.weight.dtype == torch.uint8 and native.weight.shape == (8, 128)
    x = torch.randn(2, 32, 256, device="cuda", dtype=dtype)
    with pytest.raises(RuntimeError, match="not been set"):
        native(x)
    for call in (0, 1):
        state.set(call)
        if abits == 4:  # the reference's own exact case: step sizes that are powers of two (clip / 7)
            torch.testing.assert_close(native(x), reference(x), rtol=0, atol=0)
        else:  # clip / 127 is not: the kernel multiplies where the CPU module divides; the reference's W4A8 bar
            got, want = native(x).float(), reference(x).float()  # (tests/test_w4a8.py:30: relative RMS < 0.005)
            assert ((got - want).square().mean().sqrt() / want.square().mean().sqrt()).item() < 0.005


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("m,k,n", [(32, 1024, 3072), (32, 4096, 1024), (129, 3072, 3072), (294, 3072, 14336),
                                   (294, 14336, 3072)])
def test_reference_module_on_rotated_sites(ref, dtype, m, k, n):
    """The reference module hands its signs to ``symmetric_scheduled_stream_rht_linear`` with no rotation keyword;
    the operator must apply the reference's rotation for the width (full-width transform, had12 x H256, had28 x H512)."""
    R, C, S, St, rht = ref["runtime"], ref["checkpoint"], ref["streams"], ref["state"], ref["rht"]
    torch.manual_seed(42)
    counts = (128, 1) if m == 129 else (16, 16) if m == 32 else (98, 98, 98)
    names = ("text", "proprio") if m == 129 else tuple(
        f"action_chunk_{i}" if m == 32 else f"latent_frame_{i}" for i in range(len(counts)))
    source = torch.nn.Linear(k, n, device="cuda", dtype=dtype)
    entry = C.QuantizedSite(
        0, "linear", "video" if m == 294 else "action", "cross_attn.k" if m == 129 else "self_attn.q", names,
        torch.randint(-7, 8, (n, k), dtype=torch.int8), torch.full((n, 1), 0.002), torch.linspace(0.5, 2, k),
        torch.ones(10, len(counts)), torch.linspace(2.0, 4.0, 10),
        torch.tensor(counts).float()[None].repeat(10, 1) / m, 0.0, 0.0, (0.0,) * 10, (0.0,) * 10,
        rht.rht_signs(k, seed=42, module_name="linear"), "rht")
    raw = torch.linspace(-0.4, 0.4, len(counts))
    entry.gamma_gains[:] = (raw - (raw * entry.token_fractions[0]).sum()).exp()
    state = St.DenoiseCallState(10)
    module = R.WAMQuantLinear(source, entry, state=state, stream_config=S.FastWAMStreamConfig(), weight_bits=4,
                              activation_bits=4, backend="cutlass_w4a4")
    x = torch.randn(2 if m == 129 else 1, m, k, device="cuda", dtype=dtype)

    def expected():
        z = rht.rht_transform(x.float(), module.input_rotation_signs, "rht").to(dtype).float()
        gain = torch.repeat_interleave(module.gamma_gains[state.require()], torch.tensor(counts, device="cuda"))[None, :, None]
        scale = module.clipping_ranges[state.require()]
        codes = (z * module.input_scale * (gain / scale)).round().clamp(-7, 7)
        acc = torch.nn.functional.linear(codes, entry.qweight.cuda().float())
        return (acc * (scale / gain) * module.weight_scales + source.bias.float()).to(dtype)

    with torch.inference_mode():
        for call in (0, 9):
            state.set(call)
            actual, want = module(x), expected()
            rel = (actual.float() - want.float()).square().mean().sqrt() / want.float().square().mean().sqrt()
            assert rel < 0.003, float(rel)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                captured = module(x)
            graph.replay()
            torch.testing.assert_close(captured, actual, atol=0, rtol=0)
            x.mul_(0.79)
            eager = module(x)
            graph.replay()
            torch.testing.assert_close(captured, eager, atol=0, rtol=0)


def test_reference_live_graph_replays_this_librarys_kernels(ref):
    """The reference's ``LiveJointDiTGraph`` and call tracker around a model whose denoise core is a reference
    ``WAMQuantLinear`` on the native backend: two calls -> two graphs, three different inputs -> six replays, every
    result bit-equal to the eager run (tests/test_rollout_graph.py:62-87)."""
    R, C, S, St, G = ref["runtime"], ref["checkpoint"], ref["streams"], ref["state"], ref["rollout_graph"]
    torch.manual_seed(3)
    k = n = 1024
    source = torch.nn.Linear(k, n, device="cuda", dtype=torch.bfloat16)
    entry = C.QuantizedSite(
        0, "linear", "action", "self_attn.q", ("action_chunk_0", "action_chunk_1"),
        torch.randint(-7, 8, (n, k), dtype=torch.int8), torch.full((n, 1), 0.002), torch.linspace(0.5, 2, k),
        torch.tensor([[0.5, 2.0], [2.0, 0.5]]), torch.tensor([2.0, 3.0]), torch.full((2, 2), 0.5), 0.0, 0.0,
        (0.0, 0.0), (0.0, 0.0))

    class Tiny(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.state = St.DenoiseCallState(2)
            self.layer = R.WAMQuantLinear(source, entry, state=self.state, stream_config=S.FastWAMStreamConfig(),
                                          weight_bits=4, activation_bits=8, backend="cutlass_w4a8")
            self._wam_call_tracker = St.FastWAMCallTracker(self, self.state)
            self._wam_call_tracker.install()

        def _joint_denoise_core(self, x, scale):
            y = self.layer(x) * scale
            return y, y + 1

        def _predict_joint_noise(self, **kwargs):
            return self._joint_denoise_core(**kwargs)

        @torch.no_grad()
        def infer_action(self, x, scale, num_inference_steps=2, text_cfg_scale=1.0, compile_action_infer=False):
            self._wam_call_tracker.reset()
            for _ in range(num_inference_steps):
                x, _ = self._predict_joint_noise(x=x, scale=scale)
            return x

    model = Tiny().cuda().eval()
    inputs = [dict(x=(torch.randn(1, 32, k, device="cuda") * (1 + i)).bfloat16(),
                   scale=torch.tensor(0.5 + i, device="cuda", dtype=torch.bfloat16)) for i in range(3)]
    expected = [model.infer_action(**values) for values in inputs]
    graph = G.LiveJointDiTGraph(model, num_calls=2).install()
    actual = [model.infer_action(**values) for values in inputs]
    for a, b in zip(actual, expected):
        torch.testing.assert_close(a, b, rtol=0, atol=0)
    assert len(graph.entries) == 2 and graph.replays == 6
    with pytest.raises(ValueError, match="schedule changed"):
        model.infer_action(**dict(inputs[0], num_inference_steps=3))
    graph.remove()
