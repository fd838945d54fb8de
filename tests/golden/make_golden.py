"""Generate ``steerquant_golden.npz`` by running the reference package itself.

Run where the reference checkout is available, e.g.

    python tests/golden/make_golden.py --reference /path/to/reference

It imports ``fastwam_steerquant`` from ``<reference>/src`` and records outputs of
the reference's own CPU primitives on small seeded inputs.  The resulting file
is committed; the tests that read it need neither the reference nor this script.
bfloat16 tensors are stored as their int16 bit patterns (suffix ``_bf16``).
"""
from __future__ import annotations

import argparse
import sys
from pathlib import Path

import numpy as np
import torch


def bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy()


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--reference", required=True, help="root of the reference checkout")
    parser.add_argument("--out", default=str(Path(__file__).with_name("steerquant_golden.npz")))
    args = parser.parse_args()
    sys.path.insert(0, str(Path(args.reference) / "src"))

    from fastwam_steerquant import quant, rht
    from fastwam_steerquant.checkpoint import QuantizedSite
    from fastwam_steerquant.kernels.w4a8.ops import pack_signed_int4
    from fastwam_steerquant.runtime import WAMQuantLinear
    from fastwam_steerquant.state import DenoiseCallState
    from fastwam_steerquant.streams import FastWAMStreamConfig

    out: dict[str, np.ndarray] = {}
    gen = torch.Generator(device="cpu").manual_seed(1234)

    # --- signs (rht.py:81-96)
    out["signs_64_s0_linear"] = rht.rht_signs(64, seed=0, module_name="linear").numpy()
    out["signs_256_s42_blocks0q"] = rht.rht_signs(256, seed=42, module_name="blocks.0.q").numpy()
    out["signs_3072_s0_linear_head"] = rht.rht_signs(3072, seed=0, module_name="linear")[:64].numpy()

    # --- block Hadamard (rht.py:99-112) on [..., K/128, 128] and the rotation wrappers
    x = torch.randn(5, 384, generator=gen) * 3.0
    out["had_in"] = x.numpy()
    out["had128_out"] = rht._normalized_block_hadamard(x.reshape(5, 3, 128)).reshape(5, 384).numpy()
    x256 = torch.randn(3, 256, generator=gen)
    signs256 = rht.rht_signs(256, seed=7, module_name="site")
    out["rot_in"] = x256.numpy()
    out["rot_signs"] = signs256.numpy()
    out["rot_rht_out"] = rht.rht_transform(x256, signs256, "rht").numpy()
    out["rot_block_out"] = rht.rht_transform(x256, signs256, "block").numpy()
    # the model-dtype rounding boundary used by install_rht_ (rht_install.py:46-49)
    xb = (torch.randn(4, 256, generator=gen) * 2.0).bfloat16()
    out["rot_bf16_in_bf16"] = bits(xb)
    out["rot_bf16_out_bf16"] = bits(rht.rht_transform(xb.float(), signs256, "rht").to(torch.bfloat16))

    # --- fake quant (quant.py:6-21) with per-row scales
    v = torch.randn(6, 128, generator=gen) * 4.0
    v[2] = 0.0  # all-zero row exercises the 1e-8 clamp
    for b in (8, 4):
        qmax = 2 ** (b - 1) - 1
        scale = v.abs().amax(dim=-1, keepdim=True) / qmax
        out[f"fq_in"] = v.numpy()
        out[f"fq_a{b}_out"] = quant.symmetric_fake_quant(v, bits=b, scale=scale).numpy()
        out[f"fq_a{b}_scale"] = scale.numpy()
    # ties: values exactly half way between codes must round to even
    ties = torch.tensor([[0.5, 1.5, 2.5, -0.5, -1.5, -2.5, 6.5, 7.5]])
    out["fq_ties_in"] = ties.numpy()
    out["fq_ties_out"] = quant.symmetric_fake_quant(ties, bits=4, scale=torch.ones(1, 1)).numpy()

    # --- weights (quant.py:55-64) per channel and on [N*K/128, 128] groups; packing (ops.py:8-14)
    w = torch.randn(16, 256, generator=gen) * 0.02
    qw, ws = quant.quantize_weight_per_channel(w, bits=4)
    out["w_in"] = w.numpy()
    out["w_q_channel"] = qw.numpy()
    out["w_s_channel"] = ws.numpy()
    qg, sg = quant.quantize_weight_per_channel(w.reshape(32, 128), bits=4)
    out["w_q_group_fp32scale"] = qg.reshape(16, 256).numpy()
    out["w_s_group_fp32scale"] = sg.reshape(16, 2).numpy()
    q_all = torch.randint(-8, 8, (8, 64), generator=gen, dtype=torch.int8)
    out["pack_in"] = q_all.numpy()
    out["pack_out"] = pack_signed_int4(q_all).numpy()

    # --- the reference CPU module (runtime.py:155-175), un-rotated and rotated, both calls
    for tag, rotated in (("plain", False), ("rht", True)):
        for dtype, dname in ((torch.bfloat16, "bf16"),):
            torch.manual_seed(99)
            source = torch.nn.Linear(256, 8, bias=True, dtype=dtype)
            qweight = torch.randint(-7, 8, (8, 256), generator=gen, dtype=torch.int8)
            wscale = (torch.rand(8, 1, generator=gen) * 0.01 + 0.002)
            dvec = torch.rand(256, generator=gen) + 0.5
            gains = torch.tensor([[0.5, 2.0], [2.0, 0.5]])
            clips = torch.tensor([1.75, 3.5])
            signs = rht.rht_signs(256, seed=42, module_name="linear") if rotated else None
            entry = QuantizedSite(
                0, "linear", "action", "self_attn.o", ("action_chunk_0", "action_chunk_1"),
                qweight, wscale, dvec, gains, clips, torch.full((2, 2), 0.5), 0.0, 0.0,
                (0.0, 0.0), (0.0, 0.0), signs, "rht" if rotated else "none")
            state = DenoiseCallState(2)
            for abits in (8, 4):
                module = WAMQuantLinear(source, entry, state=state, stream_config=FastWAMStreamConfig(),
                                        weight_bits=4, activation_bits=abits, backend="reference")
                xin = (torch.randn(2, 32, 256, generator=torch.Generator().manual_seed(5)) * 1.5).to(dtype)
                for call in (0, 1):
                    state.set(call)
                    with torch.no_grad():
                        y = module(xin)
                    out[f"mod_{tag}_a{abits}_call{call}_out_bf16"] = bits(y)
            out[f"mod_{tag}_x_bf16"] = bits(xin)
            out[f"mod_{tag}_qweight"] = qweight.numpy()
            out[f"mod_{tag}_wscale"] = wscale.numpy()
            out[f"mod_{tag}_d"] = dvec.numpy()
            out[f"mod_{tag}_gains"] = gains.numpy()
            out[f"mod_{tag}_clips"] = clips.numpy()
            out[f"mod_{tag}_bias_bf16"] = bits(source.bias.detach())
            if rotated:
                out[f"mod_{tag}_signs"] = signs.numpy()

    # --- the composite rotation of widths 3072 / 14336 (rht.py:18-39): the order-12 / order-28 sign matrices
    # the reference rebuilds from its pinned masks, and its transform of seeded rows
    mix_gen = torch.Generator(device="cpu").manual_seed(4321)
    for order, width, rows in ((12, 3072, 2), (28, 14336, 1)):
        out[f"mix{order}_matrix"] = rht.official_hadamard_matrix(order).to(torch.int8).numpy()
        xin = torch.randn(rows, width, generator=mix_gen) * 1.5
        signs_w = rht.rht_signs(width, seed=42, module_name="linear")
        out[f"mix{order}_in"] = xin.numpy()
        out[f"mix{order}_out"] = rht.rht_transform(xin, signs_w, "rht").numpy()
        out[f"mix{order}_out_bf16"] = bits(rht.rht_transform(xin.bfloat16().float(), signs_w, "rht").to(torch.bfloat16))

    # --- the reference CPU module on rotated sites whose rotation the width alone selects: had12 x H256 at
    # 3072 (rht.py:31-39) and the full-width transform at 1024; appended last, with generators of their own, so
    # the arrays above keep their values
    for width in (3072, 1024):
        wide_gen = torch.Generator(device="cpu").manual_seed(777 + width)
        torch.manual_seed(7)
        source = torch.nn.Linear(width, 8, bias=True, dtype=torch.bfloat16)
        qweight = torch.randint(-7, 8, (8, width), generator=wide_gen, dtype=torch.int8)
        wscale = torch.rand(8, 1, generator=wide_gen) * 0.01 + 0.002
        dvec = torch.rand(width, generator=wide_gen) + 0.5
        gains = torch.tensor([[0.5, 2.0], [2.0, 0.5]])
        clips = torch.tensor([1.75, 3.5])
        signs = rht.rht_signs(width, seed=42, module_name="linear")
        entry = QuantizedSite(0, "linear", "action", "self_attn.o", ("action_chunk_0", "action_chunk_1"), qweight,
                              wscale, dvec, gains, clips, torch.full((2, 2), 0.5), 0.0, 0.0, (0.0, 0.0), (0.0, 0.0),
                              signs, "rht")
        state = DenoiseCallState(2)
        module = WAMQuantLinear(source, entry, state=state, stream_config=FastWAMStreamConfig(), weight_bits=4,
                                activation_bits=4, backend="reference")
        xin = (torch.randn(1, 6, width, generator=wide_gen) * 1.5).bfloat16()
        tag = f"wide{width}"
        for call in (0, 1):
            state.set(call)
            with torch.no_grad():
                out[f"mod_{tag}_a4_call{call}_out_bf16"] = bits(module(xin))
        out[f"mod_{tag}_x_bf16"] = bits(xin)
        out[f"mod_{tag}_qweight"] = qweight.numpy()
        out[f"mod_{tag}_wscale"] = wscale.numpy()
        out[f"mod_{tag}_d"] = dvec.numpy()
        out[f"mod_{tag}_gains"] = gains.numpy()
        out[f"mod_{tag}_clips"] = clips.numpy()
        out[f"mod_{tag}_bias_bf16"] = bits(source.bias.detach())
        out[f"mod_{tag}_signs"] = signs.numpy()
        out[f"rot_{tag}_out_bf16"] = bits(rht.rht_transform(xin.float(), signs, "rht").to(torch.bfloat16))

    np.savez_compressed(args.out, **out)
    print(f"wrote {args.out}: {len(out)} arrays, {Path(args.out).stat().st_size} bytes")


if __name__ == "__main__":
    main()
