"""Packed deployment files and the checkpoint container, on the reference's own test cases
(tests/test_deployment.py:36-101, tests/test_deployment_aliases.py, tests/test_policy.py): a tiny model with the
FastWAM topology is exported, loaded back on ``meta`` and on CPU, and every buffer of every loaded site must equal
what ``apply_checkpoint`` builds from the same checkpoint, with atol = 0."""
import copy
import importlib
from dataclasses import asdict, replace
from types import SimpleNamespace

import pytest
import torch
from torch import nn

P = "fastwamjoint_quantization_b200."


@pytest.fixture(scope="module")
def m(pkg):
    names = ("checkpoint", "deployment", "runtime", "topology", "streams", "rht", "state", "policy")
    return SimpleNamespace(**{name: importlib.import_module(P + name) for name in names})


class Attention(nn.Module):
    def __init__(self, hidden):
        super().__init__()
        for name in "qkvo":
            setattr(self, name, nn.Linear(hidden, hidden))


class Block(nn.Module):
    def __init__(self, hidden):
        super().__init__()
        self.self_attn, self.cross_attn = Attention(hidden), Attention(hidden)
        self.ffn = nn.Sequential(nn.Linear(hidden, 2 * hidden), nn.GELU(), nn.Linear(2 * hidden, hidden))


class Expert(nn.Module):
    def __init__(self, hidden, layers):
        super().__init__()
        self.blocks = nn.ModuleList(Block(hidden) for _ in range(layers))


class TinyWAM(nn.Module):
    """Two experts of one block each: the module paths the site enumeration walks."""

    def __init__(self, hidden=256, layers=1):
        super().__init__()
        self.video_expert, self.action_expert = Expert(hidden, layers), Expert(hidden, layers)


def tiny_model(hidden=256, device="cpu"):
    with torch.device(device):
        model = TinyWAM(hidden).bfloat16()
        model.register_buffer("aux", torch.ones(3), persistent=False)
        model.extra = nn.Linear(8, 8, dtype=torch.bfloat16)
    return model


def aliased_model(device="cpu"):
    """The same experts registered a second and third time, and one Linear kept under a shortcut attribute."""
    model = tiny_model(256, device)
    model.mot = nn.Module()
    model.mot.mixtures = nn.ModuleDict({"video": model.video_expert, "action": model.action_expert})
    model.dit = model.mot
    model.shortcut = model.video_expert.blocks[0].self_attn.q
    return model


def tiny_checkpoint(m, model, bits=8, rotation="none"):
    sites = []
    for site in m.topology.enumerate_fastwamjoint_linears(model):
        n, k = site.module.weight.shape
        stream = "context" if site.stream_kind == "context" else (
            "latent_frame_0" if site.expert == "video" else "action_chunk_0")
        signs = m.rht.rht_signs(k, seed=42, module_name=site.module_name) if rotation == "rht" else None
        sites.append(m.checkpoint.QuantizedSite(
            site.index, site.module_name, site.expert, site.operation, (stream,),
            torch.randint(-7, 8, (n, k), dtype=torch.int8), torch.full((n, 1), 0.002), torch.linspace(0.7, 1.4, k),
            torch.ones(2, 1), torch.tensor([2.0, 3.0]), torch.ones(2, 1), 0.0, 0.0, (0.0, 0.0), (0.0, 0.0), signs,
            rotation))
    streams = asdict(m.streams.FastWAMStreamConfig(video_latent_frames=1, action_chunks=1, split_context=False))
    return m.checkpoint.QuantizationCheckpoint(4, bits, 2, streams, {"epochs": 1}, {"epochs": 1}, tuple(sites))


@pytest.mark.parametrize("bits,rotation", [(8, "none"), (4, "none"), (4, "rht")])
@pytest.mark.parametrize("construct_device", ["meta", "cpu"])
def test_export_then_direct_load_equals_apply_checkpoint(m, tmp_path, bits, rotation, construct_device):
    torch.manual_seed(5)
    original = tiny_model()
    checkpoint = tiny_checkpoint(m, original, bits, rotation)
    path = m.deployment.export_deployment(original, checkpoint, tmp_path / "deploy.pt", model_config={"hidden": 256})
    built_on = []

    def builder(config, *, device):
        built_on.append(device)
        return tiny_model(config["hidden"], device)

    loaded, state, metadata = m.deployment.load_deployment(path, builder, device="cpu",
                                                           construct_device=construct_device)
    assert built_on == [construct_device]
    assert state.num_calls == 2 and metadata["activation_bits"] == bits and "state_dict" not in metadata
    torch.testing.assert_close(loaded.aux, original.aux)
    torch.testing.assert_close(loaded.extra.weight, original.extra.weight)
    replaced = copy.deepcopy(original)
    m.runtime.apply_checkpoint(replaced, checkpoint, backend=f"cutlass_w4a{bits}")
    for entry in checkpoint.sites:
        direct = m.topology.resolve_site_module(loaded, entry.module_name)
        via_checkpoint = m.topology.resolve_site_module(replaced, entry.module_name)
        assert isinstance(direct, m.runtime.WAMQuantLinear) and direct.weight.dtype == torch.uint8
        assert direct.weight.numel() * 2 == entry.qweight.numel()
        assert not list(direct.parameters())  # no floating-point source weight is retained
        assert set(direct.state_dict()) == set(via_checkpoint.state_dict())
        for name, value in via_checkpoint.state_dict().items():
            torch.testing.assert_close(direct.state_dict()[name], value, rtol=0, atol=0)
        if rotation == "rht":  # both routes pick the reference's rotation for K = 256 / 512 from the width alone
            assert direct.official_rotation and via_checkpoint.official_rotation
            assert direct.rotation_block == via_checkpoint.rotation_block
            for a, b in ((direct.rotation_matrix, via_checkpoint.rotation_matrix),):
                assert (a is None) == (b is None) and (a is None or torch.equal(a, b))
    assert all(t.device.type == "cpu" for t in (*loaded.parameters(), *loaded.buffers()))


def test_export_refuses_partial_checkpoints_and_overwriting(m, tmp_path):
    model = tiny_model(32)
    checkpoint = tiny_checkpoint(m, model)
    with pytest.raises(ValueError, match="every target"):
        m.deployment.export_deployment(model, replace(checkpoint, sites=checkpoint.sites[:1]), tmp_path / "x.pt",
                                       model_config={})
    path = m.deployment.export_deployment(model, checkpoint, tmp_path / "x.pt", model_config={})
    with pytest.raises(FileExistsError):
        m.deployment.export_deployment(model, checkpoint, path, model_config={})
    with pytest.raises(ValueError, match="meta or CPU"):
        m.deployment.load_deployment(path, lambda cfg, device: tiny_model(32, device), construct_device="cuda")


def test_payload_checks_and_wrong_builder(m, tmp_path):
    model = tiny_model(32)
    path = m.deployment.export_deployment(model, tiny_checkpoint(m, model), tmp_path / "x.pt", model_config={})
    payload = torch.load(path, weights_only=True)
    m.deployment.validate_payload(payload)
    key = payload["sites"][0]["module_name"] + ".weight"
    unpacked = dict(payload, state_dict=dict(payload["state_dict"]))
    unpacked["state_dict"][key] = payload["state_dict"][key].to(torch.int8)
    with pytest.raises(ValueError, match="packed uint8"):
        m.deployment.validate_payload(unpacked)
    with pytest.raises(ValueError, match="Unsupported deployment format"):
        m.deployment.validate_payload(dict(payload, format="something_else"))
    negative = dict(payload, state_dict=dict(payload["state_dict"]))
    scale_key = payload["sites"][0]["module_name"] + ".weight_scales"
    negative["state_dict"][scale_key] = -payload["state_dict"][scale_key]
    with pytest.raises(ValueError, match="Nonpositive"):
        m.deployment.validate_payload(negative)
    with pytest.raises(ValueError, match="shape/bias"):
        m.deployment.load_deployment(path, lambda cfg, device: tiny_model(64, device), device="cpu")


@pytest.mark.parametrize("bits,rotation", [(8, "none"), (4, "rht")])
@pytest.mark.parametrize("construct_device", ["cpu", "meta"])
def test_aliased_experts_are_stored_once_and_load_strictly(m, tmp_path, bits, rotation, construct_device):
    model = aliased_model()
    untouched = model.shortcut.weight.clone()
    checkpoint = tiny_checkpoint(m, model, bits, rotation)
    path = m.deployment.export_deployment(model, checkpoint, tmp_path / "deploy.pt", model_config={})
    payload = torch.load(path, weights_only=True)
    for spec in payload["sites"]:
        assert len(spec["aliases"]) >= 3
        canonical = payload["state_dict"][spec["module_name"] + ".weight"]
        assert canonical.dtype == torch.uint8
        assert all(payload["state_dict"][alias + ".weight"] is canonical for alias in spec["aliases"])
    torch.testing.assert_close(model.shortcut.weight, untouched, rtol=0, atol=0)  # export does not modify the model
    loaded, _, _ = m.deployment.load_deployment(path, lambda cfg, device: aliased_model(device), device="cpu",
                                                construct_device=construct_device)
    assert loaded.dit is loaded.mot and loaded.mot.mixtures.video is loaded.video_expert
    assert loaded.shortcut is loaded.video_expert.blocks[0].self_attn.q
    for spec in payload["sites"]:
        module = m.topology.resolve_site_module(loaded, spec["module_name"])
        assert isinstance(module, m.runtime.WAMQuantLinear) and not list(module.parameters())
        assert module.weight.dtype == torch.uint8 and module.weight_scales.dtype == torch.float32
        assert all(m.topology.resolve_site_module(loaded, alias) is module for alias in spec["aliases"])
        for name, value in module.state_dict().items():
            torch.testing.assert_close(value, payload["state_dict"][spec["module_name"] + "." + name], rtol=0, atol=0)


@pytest.mark.parametrize("damage", ["missing", "bf16", "different_value", "duplicate", "overlap"])
def test_alias_conflicts_are_refused(m, tmp_path, damage):
    model = aliased_model()
    path = m.deployment.export_deployment(model, tiny_checkpoint(m, model), tmp_path / "deploy.pt", model_config={})
    payload = torch.load(path, weights_only=True)
    spec = payload["sites"][0]
    alias = next(a for a in spec["aliases"] if a != spec["module_name"])
    key = alias + ".weight"
    if damage == "missing":
        del payload["state_dict"][key]
    elif damage == "bf16":
        payload["state_dict"][key] = torch.ones(spec["out_features"], spec["in_features"], dtype=torch.bfloat16)
    elif damage == "different_value":
        payload["state_dict"][key] = payload["state_dict"][key].clone()
        payload["state_dict"][key][0, 0] ^= 1
    elif damage == "duplicate":
        spec["aliases"].append(alias)
    else:
        payload["sites"][1]["aliases"].append(alias)
    with pytest.raises(ValueError, match="alias"):
        m.deployment.validate_payload(payload)


def test_builder_with_a_different_alias_graph_and_files_without_aliases(m, tmp_path):
    model = aliased_model()
    path = m.deployment.export_deployment(model, tiny_checkpoint(m, model), tmp_path / "deploy.pt", model_config={})

    def other_graph(cfg, *, device):
        result = aliased_model(device)
        result.shortcut = copy.deepcopy(result.shortcut)
        return result

    with pytest.raises(ValueError, match="alias topology"):
        m.deployment.load_deployment(path, other_graph, device="cpu")
    plain = tiny_model(32)
    plain_path = m.deployment.export_deployment(plain, tiny_checkpoint(m, plain), tmp_path / "plain.pt", model_config={})
    payload = torch.load(plain_path, weights_only=True)
    for spec in payload["sites"]:
        del spec["aliases"]  # a v1 file written before aliases were recorded
    torch.save(payload, tmp_path / "legacy.pt")
    m.deployment.load_deployment(tmp_path / "legacy.pt", lambda cfg, device: tiny_model(32, device), device="cpu")


def test_checkpoint_container_round_trip_merge_and_refusals(m, tmp_path):
    model = tiny_model(32)
    for rotation, fmt in (("none", "fastwam_steerquant_calibration_v1"), ("rht", "fastwam_steerquant_calibration_rht_v1")):
        checkpoint = tiny_checkpoint(m, model, 4, rotation)
        assert checkpoint.state_dict()["format"] == fmt
        back = m.checkpoint.QuantizationCheckpoint.load(checkpoint.save(tmp_path / f"{rotation}.pt"))
        assert back.num_calls == 2 and len(back.sites) == len(checkpoint.sites)
        for a, b in zip(back.sites, checkpoint.sites):
            assert a.module_name == b.module_name and a.stream_names == b.stream_names and a.rotation == b.rotation
            assert torch.equal(a.qweight, b.qweight) and torch.equal(a.gamma_gains, b.gamma_gains)
            assert (a.input_rotation_signs is None) == (b.input_rotation_signs is None)
    checkpoint = tiny_checkpoint(m, model)
    halves = replace(checkpoint, sites=checkpoint.sites[:7]), replace(checkpoint, sites=checkpoint.sites[7:])
    merged = m.checkpoint.QuantizationCheckpoint.merge(reversed(halves))
    assert [s.site_index for s in merged.sites] == list(range(len(checkpoint.sites)))
    with pytest.raises(ValueError, match="overlap"):
        m.checkpoint.QuantizationCheckpoint.merge((halves[0], halves[0]))
    with pytest.raises(ValueError, match="do not match"):
        m.checkpoint.QuantizationCheckpoint.merge((halves[0], replace(halves[1], d_config={"epochs": 2})))
    mixed = replace(checkpoint, sites=(checkpoint.sites[0], replace(
        checkpoint.sites[1], rotation="rht", input_rotation_signs=torch.ones(checkpoint.sites[1].qweight.shape[1]))))
    with pytest.raises(ValueError, match="mix rotated"):
        mixed.validate()
    wrong_tag = checkpoint.state_dict()
    wrong_tag["format"] = "fastwam_steerquant_calibration_rht_v1"
    with pytest.raises(ValueError, match="disagree"):
        m.checkpoint.QuantizationCheckpoint.from_state_dict(wrong_tag)


class FakeModel(nn.Module):
    """``infer_action`` calls ``_predict_joint_noise`` once per step; the value returned counts the call indices."""

    def __init__(self):
        super().__init__()
        self.fail_once = False

    def _predict_joint_noise(self, value):
        if self.fail_once:
            self.fail_once = False
            raise RuntimeError("interrupted chunk")
        return value + self._wam_call_tracker.state.require()

    def infer_action(self, *, num_inference_steps, **kwargs):
        value = torch.zeros(1)
        for _ in range(num_inference_steps):
            value = self._predict_joint_noise(value)
        return {"action": value}


def fake_policy(m, monkeypatch):
    model, state = FakeModel(), m.state.DenoiseCallState(2)
    metadata = {"model_config": {"sigma_shift": None, "model": {"action_horizon": 4, "num_video_frames": 5}}}
    monkeypatch.setattr(m.policy, "load_deployment", lambda *a, **kw: (model, state, metadata))
    adapter = SimpleNamespace(
        build_model=lambda *a, **kw: model,
        infer_kwargs=lambda model, record, seed: {"num_inference_steps": record.get("steps", 2),
                                                  "action_horizon": record.get("horizon", 4), "num_video_frames": 5})
    return m.policy.QuantizedPolicy("fixture", adapter, device="cpu", cuda_graph=False)


def test_policy_clears_the_call_state_between_chunks_and_after_an_error(m, monkeypatch):
    policy = fake_policy(m, monkeypatch)
    for _ in range(3):
        torch.testing.assert_close(policy.infer({})["action"], torch.ones(1))  # calls 0 and 1: 0 + 1
        assert policy.state.index is None
    policy.model.fail_once = True
    with pytest.raises(RuntimeError, match="interrupted"):
        policy.infer({})
    assert policy.state.index is None
    torch.testing.assert_close(policy.infer({})["action"], torch.ones(1))


def test_policy_refuses_other_geometry_and_reentrant_calls(m, monkeypatch):
    policy = fake_policy(m, monkeypatch)
    with pytest.raises(ValueError, match="num_inference_steps"):
        policy.infer({"steps": 3})
    with pytest.raises(ValueError, match="action_horizon"):
        policy.infer({"horizon": 8})
    policy._busy.acquire()
    try:
        with pytest.raises(RuntimeError, match="serialized"):
            policy.infer({})
    finally:
        policy._busy.release()
    with pytest.raises(ValueError, match="explicitly support"):
        m.policy.QuantizedPolicy("fixture", policy.adapter, device="cpu", cuda_graph=False, fuse_block=True)


@pytest.mark.gpu
@pytest.mark.parametrize("bits,rotation", [(8, "none"), (4, "rht")])
def test_directly_loaded_model_computes_what_the_replaced_model_computes(m, tmp_path, bits, rotation):
    """tests/test_deployment.py:86-101: outputs of every site, loaded straight from the file onto the GPU, against
    the same site after ``apply_checkpoint`` on the GPU, atol = rtol = 0."""
    original = tiny_model()
    checkpoint = tiny_checkpoint(m, original, bits, rotation)
    path = m.deployment.export_deployment(original, checkpoint, tmp_path / "gpu.pt", model_config={})
    direct, direct_state, _ = m.deployment.load_deployment(path, lambda cfg, device: tiny_model(device=device))
    replaced = original.cuda()
    replaced_state, _ = m.runtime.apply_checkpoint(replaced, checkpoint, backend=f"cutlass_w4a{bits}")
    for call in (0, 1):
        direct_state.set(call)
        replaced_state.set(call)
        for entry in checkpoint.sites:
            x = torch.randn(1, 6, entry.qweight.shape[1], device="cuda", dtype=torch.bfloat16)
            a = m.topology.resolve_site_module(direct, entry.module_name)(x)
            b = m.topology.resolve_site_module(replaced, entry.module_name)(x)
            torch.testing.assert_close(a, b, atol=0, rtol=0)
