"""Benchmark of the quantized-linear hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2|c1|...] [--impl b200|reference]

One step = one pass of the hot path (activation pre-pass + W4 GEMM with fused epilogue)
over one batch of seeded synthetic input.  The default workload is the configuration the
headline metric is quoted on: a single W4A4+RHT linear, M=2048, K=3072, N=3072, group-128
fp16 weight scales, per-token int4 activations, 128-point randomized Hadamard transform.
Prints ONE JSON line (rank 0).  Multi-GPU runs shard tokens (M) across ranks with replicated
weights and no collective: every rank runs the per-GPU workload, so scaling is "weak".
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

WORKLOADS = {
    # name: (M, K, N, activation bits, rotate)
    "c1": (256, 1024, 1024, 8, False),
    "c2": (2048, 3072, 3072, 4, True),
    "c2_a8": (2048, 3072, 3072, 8, False),
    "m4096_ffn_up": (4096, 3072, 12288, 4, True),
    "m4096_ffn_down": (4096, 12288, 3072, 4, True),
    "m16384": (16384, 3072, 3072, 4, True),
}
L2_BYTES = 126 * 1024 * 1024


def algorithmic_bytes(m, k, n, rotate):
    """What one linear has to move whatever form the kernel reads: bf16 x + packed int4 weights + fp16 group
    scales + bias + bf16 out (+ fp32 signs)."""
    return 2 * m * k + n * k // 2 + 2 * n * (k // 128) + 2 * n + 2 * m * n + (4 * k if rotate else 0)


def load_oracle():
    sys.path.insert(0, str(ROOT / "oracle"))
    import steerquant_oracle
    return steerquant_oracle


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU through NVML (read-only) every 100 ms."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index: int):
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.max_mhz = index, [], set(), None
        self._halt = threading.Event()
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nvml = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
        except Exception:  # no NVML: report empty clocks rather than fail the bench
            self.nvml = None

    def run(self):
        while self.nvml is not None and not self._halt.is_set():
            try:
                self.samples.append(self.nvml.nvmlDeviceGetClockInfo(self.handle, self.nvml.NVML_CLOCK_SM))
                mask = self.nvml.nvmlDeviceGetCurrentClocksEventReasons(self.handle)
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._halt.wait(0.1)

    def stop(self):
        self._halt.set()
        self.join(timeout=2)
        mid = sorted(self.samples)[len(self.samples) // 2] if self.samples else None
        return {"sm_mhz": mid, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}


def cpu_forward_factory(oracle, case):
    """The reference's CPU arithmetic for this scheme: fake-quantize the (rotated) activation,
    one bf16 F.linear against the dequantized weight (runtime.py:155-175)."""
    def run():
        return oracle.token_module_forward(case["x"], case["qweight"], case["weight_scales"], case["bias"],
                                           abits=case["abits"], signs=case["signs"])
    return run


def time_cpu(run, seconds_budget=20.0, min_repeats=3, max_repeats=30):
    run()  # warm-up
    times = []
    start = time.perf_counter()
    while len(times) < min_repeats or (time.perf_counter() - start < seconds_budget and len(times) < max_repeats):
        t0 = time.perf_counter()
        run()
        times.append(time.perf_counter() - t0)
    times.sort()
    return times[len(times) // 2], len(times)


def run_reference(args, m, k, n, abits, rotate):
    """--impl reference: the CPU port of the reference's fake-quant path on all host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    oracle = load_oracle()
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    case = oracle.prepare_token_linear(m, k, n, abits=abits, seed=0)
    run = cpu_forward_factory(oracle, case)
    for _ in range(max(1, min(args.warmup, 2))):
        run()
    steps = max(1, min(args.steps, 20))
    t0 = time.perf_counter()
    for _ in range(steps):
        run()
    elapsed = time.perf_counter() - t0
    tops = 2.0 * m * n * k * steps / elapsed / 1e12
    line = {
        "impl": "reference", "metric": "W4A%d%s GEMM int-TOPS" % (abits, "+RHT" if rotate else ""),
        "value": tops, "unit": "TOPS", "n_gpus": args.gpus, "steps": steps, "warmup": args.warmup,
        "ms_per_step": elapsed / steps * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16 (CPU fake-quant)", "data": "synthetic",
        "config": {"workload": args.workload, "M": m, "K": k, "N": n, "abits": abits, "rht": rotate},
        "cpu_baseline": {"value": tops, "unit": "TOPS", "cores": cores, "kind": "port",
                         "sample": "%d full passes of the workload" % steps},
        "e2e": {"value": tops, "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def measure_int8_peak(device):
    """Dense int8 tensor-core peak the way the bf16 peak was measured: torch._int_mm 8192^3, best of 10."""
    a = torch.randint(-8, 8, (8192, 8192), device=device, dtype=torch.int8)
    b = torch.randint(-8, 8, (8192, 8192), device=device, dtype=torch.int8).t()
    for _ in range(3):
        torch._int_mm(a, b)
    best = float("inf")
    for _ in range(10):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        torch._int_mm(a, b)
        e1.record()
        e1.synchronize()
        best = min(best, e0.elapsed_time(e1))
    return 2.0 * 8192 ** 3 / (best * 1e-3) / 1e12


DIT_WORKLOADS = {"dit_a8": (8, False), "dit_a4": (4, True)}


def measured_peaks():
    """(HBM GB/s, source) from MEASURED_PEAKS.json, else the documented fallback."""
    peaks_file = ROOT / "MEASURED_PEAKS.json"
    if peaks_file.exists():
        return float(json.loads(peaks_file.read_text()).get("hbm_gbs", 6650.0)), "MEASURED_PEAKS.json"
    return 6650.0, "fallback"


def _time_graph(fn, reps):
    """Average milliseconds of fn() over one CUDA-graph replay of `reps` calls (CUDA events)."""
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(reps):
            fn()
    graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    graph.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps


def run_sweep(args):
    """BASELINE.json config 5: M in {16 .. 32768} x three layer shapes x (W4A8, W4A4+RHT), group-128 scales,
    per-token activation scales; whole linear (pre-pass + GEMM), one input set per case (the working set of the
    large cases exceeds L2 by itself, the small ones are latency-bound).  One JSON line with every case."""
    import __graft_entry__ as entry
    entry.load_package()
    from fastwamjoint_quantization_b200 import native
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    int8_peak = measure_int8_peak(device)
    hbm_peak, _ = measured_peaks()
    gen = torch.Generator(device=device).manual_seed(0)
    cases = []
    for abits in (8, 4):
        for (k, n) in ((3072, 3072), (3072, 12288), (12288, 3072)):
            packed = torch.randint(0, 256, (n, k // 2), device=device, dtype=torch.uint8, generator=gen)
            tiled = native.prepack_weights(packed) if args.weights == "prepacked" else None
            scales = (torch.rand(n, k // 128, device=device, generator=gen) * 0.01 + 0.001).half()
            signs = ((torch.randint(0, 2, (k,), device=device, generator=gen) * 2 - 1).float() if abits == 4 else None)
            for m in (16, 64, 256, 1024, 4096, 16384, 32768):
                x = torch.randn(m, k, device=device, generator=gen).bfloat16()
                out = torch.empty(m, n, device=device, dtype=torch.bfloat16)
                lib = native._lib.load_library()
                # room for the K-split scratch too: with few tiles (small M) the kernel splits a tile's K blocks
                work = torch.empty(lib.sq_workspace_bytes(m, k) + lib.sq_split_workspace_bytes(m), device=device, dtype=torch.uint8)
                weight = tiled if tiled is not None and m >= 512 else packed  # the int8 copy only pays above the ridge
                ms = _time_graph(lambda: native.linear(x, weight, scales, None, abits=abits, mode="token", signs=signs,
                                                       out=out, workspace=work), 20 if m <= 4096 else 5)
                ops = 2.0 * m * n * k
                roof_ms = max(ops / (int8_peak * 1e12), algorithmic_bytes(m, k, n, abits == 4) / (hbm_peak * 1e9)) * 1e3
                cases.append({"abits": abits, "rht": abits == 4, "M": m, "K": k, "N": n, "us": round(ms * 1e3, 2),
                              "tops": round(ops / ms / 1e9, 1), "frac": round(roof_ms / ms, 3)})
                del x, out, work
    status = native.device_status()
    if status != 0:
        raise SystemExit(f"device status {status}")
    best = max(c["tops"] for c in cases)
    print(json.dumps({"metric": "W4 linear int-TOPS, config-5 sweep (best case)", "value": best, "unit": "TOPS", "n_gpus": 1,
                      "steps": 1, "warmup": 3, "ms_per_step": None, "higher_is_better": True, "scaling": "weak",
                      "vs_baseline": None, "dtype": "int8 x int4 -> int32", "data": "synthetic",
                      "config": {"workload": "c5_sweep", "weights": args.weights, "weight_scales": "fp16 group-128",
                                 "activation_scales": "per-token", "int8_peak_tops": round(int8_peak, 1),
                                 "hbm_peak_gbs": hbm_peak},
                      "sweep": cases}), flush=True)


def run_channel(args):
    """The reference's production scheme on one layer shape: static D / gain / clip schedule, per-channel fp32
    weight scales, int4 activations (runtime.py:138-175; kernels w4a4.cu).  GEMM kernel alone and whole linear."""
    import __graft_entry__ as entry
    entry.load_package()
    from fastwamjoint_quantization_b200 import native
    oracle = load_oracle()
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    m, k, n = 4096, 3072, 12288
    gen = torch.Generator().manual_seed(0)
    x = (torch.randn(1, m, k, generator=gen) * 0.5).bfloat16()
    qw = torch.randint(-7, 8, (n, k), generator=gen, dtype=torch.int8)
    ws = torch.full((n,), 1 / 512)
    inverse = torch.pow(2.0, torch.randint(-1, 2, (k,), generator=gen).float())
    counts = (m // 2, m // 2)
    gains = torch.tensor([[0.5, 2.0], [2.0, 0.5]])
    act = torch.tensor([0.125, 0.25])
    packed = oracle.pack_signed_int4(qw).to(device)
    weight = native.prepack_weights(packed) if args.weights == "prepacked" else packed
    xd, wsd, invd, actd, gaind = (t.to(device) for t in (x, ws, inverse, act, gains))
    out = torch.empty(1, m, n, device=device, dtype=torch.bfloat16)
    work = torch.empty(native._lib.load_library().sq_workspace_bytes(m, k), device=device, dtype=torch.uint8)
    step = lambda: native.linear(xd, weight, wsd, None, abits=4, mode="static", inverse=invd, act_scales=actd,
                                 gains=gaind, call=1, span=counts[0], streams=2, out=out, workspace=work)
    got = step()
    rows = 64
    want = oracle.linear_static(x[:, :rows], qw, ws, None, inverse, act, gains, (rows, 0), 1, abits=4)["out"]
    if not torch.equal(got[:, :rows].cpu(), want):
        raise SystemExit("per-channel static linear differs from the kernel-order oracle (expected bit equality)")
    codes, row_scales = native.prepass(xd, abits=4, mode="static", inverse=invd, act_scale=actd[1:], gains=gaind[1],
                                       span=counts[0], streams=2)
    gemm = lambda: native.gemm(codes, weight, wsd, row_scales, None, out_dtype=torch.bfloat16, out=out.view(m, n),
                               int4_range=True)
    int8_peak = measure_int8_peak(device)
    sampler = ClockSampler(0)
    sampler.start()
    step_ms = _time_graph(step, args.steps)
    gemm_ms = _time_graph(gemm, args.steps)
    clocks = sampler.stop()
    ops = 2.0 * m * n * k
    print(json.dumps({"metric": "W4A4 per-channel static linear int-TOPS", "value": ops / step_ms / 1e9, "unit": "TOPS",
                      "n_gpus": 1, "steps": args.steps, "warmup": 3, "ms_per_step": step_ms, "higher_is_better": True,
                      "scaling": "weak", "vs_baseline": None, "dtype": "int8 x int4 -> int32", "data": "synthetic",
                      "config": {"workload": "m4096_ffn_up_channel", "M": m, "K": k, "N": n, "abits": 4,
                                 "weight_scales": "fp32 per channel", "activation_scales": "static schedule, two streams",
                                 "weights": args.weights, "l2": "inputs of one step (65 MB) + outputs (100 MB) > 126 MB L2",
                                 "launch": "the K steps are replayed as one CUDA graph"},
                      "gpu_launches": 2 * args.steps,
                      "roofline": {"bound": "tensor", "achieved": ops / gemm_ms / 1e9, "peak": int8_peak, "unit": "TOP/s",
                                   "frac": ops / gemm_ms / 1e9 / int8_peak, "traffic": None, "kernel": "sq_gemm_tc_kernel",
                                   "gemm_ms": gemm_ms},
                      "clocks": clocks, "parity": "bit-equal to the kernel-order oracle on the checked rows"}), flush=True)


def run_nsplit(args):
    """Output-channel split of the widest layer (3072 -> 12288, W4A4+RHT, M = 4096 tokens on every rank): rank r
    holds W[r*N/G:(r+1)*N/G], computes [M, N/G] and the slices are all-gathered with NCCL over NVLink.  The
    gather moves 2*M*N*(G-1)/G bytes per rank and dominates the step; reported as measured."""
    import torch.distributed as dist
    rank, local_rank, world = (int(os.environ.get(k, d)) for k, d in (("RANK", "0"), ("LOCAL_RANK", "0"), ("WORLD_SIZE", "1")))
    if args.impl == "reference":
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": "the reference has no multi-GPU path; use --workload m4096_ffn_up"}), flush=True)
        return
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    else:
        dist.init_process_group("nccl", init_method="tcp://127.0.0.1:29531", rank=0, world_size=1, device_id=device)
    import __graft_entry__ as entry
    entry.load_package()
    from fastwamjoint_quantization_b200 import native, sharding
    oracle = load_oracle()
    m, k, n = 4096, 3072, 12288
    case = oracle.prepare_token_linear(m, k, n, abits=4, seed=0)
    c0, c1 = sharding.channel_range(n, rank, world)
    packed = oracle.pack_signed_int4(case["qweight"][c0:c1].contiguous()).to(device)
    scales = case["weight_scales"][c0:c1].contiguous().to(device)
    x, signs = case["x"].to(device), case["signs"].to(device)
    local = lambda t: native.linear(t, packed, scales, None, abits=4, mode="token", signs=signs)
    step = lambda: sharding.channel_split_linear(x, local, chunks=args.chunks)
    serial = lambda: sharding.channel_split_linear(x, local, chunks=1)
    out = step()
    want = oracle.linear_token(case["x"][:32], case["qweight"], case["weight_scales"], None, abits=4, signs=case["signs"],
                               want_accumulators=False)["out"]
    err = ((out[:32].cpu().float() - want.float()).norm() / want.float().norm()).item()
    if not err < 1e-2:
        raise SystemExit(f"gathered output differs from the oracle: {err}")
    for _ in range(max(args.warmup, 3)):
        step()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    dist.barrier()
    # the same without overlap (one all-gather behind the whole GEMM) and the local GEMM alone, for comparison
    def timed(fn):
        for _ in range(3):
            fn()
        dist.barrier()
        torch.cuda.synchronize()
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a0.record()
        for _ in range(args.steps):
            fn()
        a1.record()
        torch.cuda.synchronize()
        dist.barrier()
        return a0.elapsed_time(a1) / args.steps

    serial_ms, local_ms = timed(serial), timed(lambda: local(x))
    # the gather fused into the GEMM: every rank's epilogue stores its block of columns into the [M, N] matrix of
    # every rank through peer pointers (sq_gemm_scatter); no collective, no re-layout
    shared = sharding.PeerMatrix(m, n, torch.bfloat16)
    codes_buf = (torch.empty((m, k), device=device, dtype=torch.int8), torch.empty((m,), device=device, dtype=torch.float32))
    fused = lambda: sharding.channel_split_linear_fused(x, packed, scales, None, shared, abits=4, signs=signs,
                                                        workspace=codes_buf)
    fused()
    torch.cuda.synchronize()
    dist.barrier()
    fused_err = ((shared.local()[:32].cpu().float() - want.float()).norm() / want.float().norm()).item()
    if not fused_err < 1e-2:
        raise SystemExit(f"fused channel-split output differs from the oracle: {fused_err}")
    fused_ms = timed(fused)
    t = torch.tensor([e0.elapsed_time(e1) / args.steps, serial_ms, local_ms, fused_ms], device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    nccl_ms, serial_ms, local_ms, fused_ms = t.tolist()
    shared.close()
    ms = fused_ms
    gather_bytes = 2 * m * n * (world - 1) // world  # bytes every rank receives per step
    if rank == 0:
        print(json.dumps({
            "metric": "W4A4+RHT GEMM int-TOPS", "value": 2.0 * m * n * k / (ms * 1e-3) / 1e12, "unit": "TOPS",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "int8 x int4 -> int32",
            "data": "synthetic",
            "config": {"workload": "nsplit_ffn_up", "M": m, "K": k, "N": n,
                       "split": "output channels across ranks; the GEMM epilogue stores its columns into every rank's "
                                "[M, N] matrix through peer pointers (no collective)",
                       "gather_bytes_per_rank": gather_bytes},
            "gpu_launches": 2 * args.steps, "parity_rel_fro": fused_err,
            "nsplit": {"ms_fused_peer_stores": fused_ms, "ms_nccl_all_gather_%d_chunks_overlapped" % args.chunks: nccl_ms,
                       "ms_nccl_all_gather_serial": serial_ms, "ms_local_gemm_only": local_ms,
                       "nccl_parity_rel_fro": err,
                       "nvlink_gbs_per_rank_out": gather_bytes / (fused_ms * 1e-3) / 1e9,
                       "transfer_ms_at_770_gbs": gather_bytes / 770e9 * 1e3,
                       "frac_of_slower_bound": max(gather_bytes / 770e9 * 1e3, 2.0 * m * (n // world) * k / 3.1e15 * 1e3) / fused_ms}}), flush=True)
    dist.destroy_process_group()


def run_dit(args):
    """30-block synthetic DiT step (BASELINE.json configs 3 / 4): hidden 3072, 24 heads, FFN 12288, 1592 tokens,
    every linear quantized, one denoising step captured and replayed as one CUDA graph.  Reports ms per step
    (lower is better).  Every GPU of a multi-GPU run holds a full replica (a batch-1 step does not shard)."""
    abits, rotate = DIT_WORKLOADS[args.workload]
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        if rank != 0:
            return
        import __graft_entry__ as entry
        entry.load_package()
        from fastwamjoint_quantization_b200 import dit
        cores = os.cpu_count() or 1
        torch.set_num_threads(cores)
        sample = 1  # blocks timed on the CPU; the step is 30 identical blocks
        cfg = dit.DiTConfig(blocks=sample, activation_bits=abits, rotate=rotate)
        model = dit.SyntheticDiT(cfg, device="cpu", backend="reference")
        x = torch.randn(1, cfg.tokens, cfg.hidden, generator=torch.Generator().manual_seed(0)).bfloat16()
        with torch.no_grad():
            model(x)
            t0 = time.perf_counter()
            model(x)
            seconds = time.perf_counter() - t0
        ms = seconds * 1e3 * 30 / sample
        print(json.dumps({
            "impl": "reference", "metric": "30-block quant DiT step ms (graph)", "value": ms, "unit": "ms",
            "n_gpus": args.gpus, "steps": 1, "warmup": 1, "ms_per_step": ms, "higher_is_better": False,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16 (CPU fake-quant)", "data": "synthetic",
            "config": {"workload": args.workload, "blocks": 30, "hidden": 3072, "ffn": 12288, "tokens": 1592},
            "cpu_baseline": {"value": ms, "unit": "ms", "cores": cores, "kind": "port",
                             "sample": "1 of 30 identical blocks timed once after one warm-up, x 30"},
            "e2e": {"value": ms, "unit": "ms", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}), flush=True)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the B200 path has no CPU fallback.")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)
    import __graft_entry__ as entry
    entry.load_package()
    from fastwamjoint_quantization_b200 import dit, native
    cfg = dit.DiTConfig(activation_bits=abits, rotate=rotate)
    model = dit.SyntheticDiT(cfg, device=device, backend="native")
    if args.weights == "prepacked":
        model.prepack()
    x = torch.randn(1, cfg.tokens, cfg.hidden, generator=torch.Generator(device=device).manual_seed(0),
                    device=device).bfloat16()
    x_host = x.cpu().pin_memory()
    out_host = torch.empty_like(x_host).pin_memory()
    with torch.no_grad():
        # parity of what is timed: the whole stack against its fake-quant reference backend, block by block -
        # teacher-forced (the kernels' own error: every block starts from the reference's activations), free-running
        # (what the stack does to earlier differences) and the fraction of activation codes that differ
        parity = dit.stack_parity(model, x)
        err = parity["output"]["linear_max"]
        if not err < 1e-2:
            raise SystemExit(f"a DiT linear differs from the fake-quant backend: relative Frobenius error {err}")
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(max(args.warmup, 3)):
                model(x)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            captured = model(x)
        graph.replay()
        torch.cuda.synchronize()
        sampler = ClockSampler(local_rank)
        sampler.start()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        ms = e0.elapsed_time(e1) / args.steps
        h0, h1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e2e_steps = max(3, min(args.steps, 20))
        h0.record()
        for _ in range(e2e_steps):
            x.copy_(x_host, non_blocking=True)
            graph.replay()
            out_host.copy_(captured, non_blocking=True)
        h1.record()
        torch.cuda.synchronize()
        e2e_ms = h0.elapsed_time(h1) / e2e_steps
    clocks = sampler.stop()
    status = native.device_status()
    if status != 0:
        raise SystemExit(f"a kernel gave up a bounded wait: device status {status}")
    if world > 1:
        t = torch.tensor([ms, e2e_ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms = t.tolist()
    if rank == 0:
        linear_ops = 2.0 * cfg.tokens * 30 * (3072 * 9216 + 3072 * 3072 + 2 * 3072 * 12288)
        print(json.dumps({
            "metric": "30-block quant DiT step ms (graph)", "value": ms, "unit": "ms", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": False,
            "scaling": "weak", "vs_baseline": None, "dtype": "int8 x int4 -> int32 linears, bf16 attention",
            "data": "synthetic",
            "config": {"workload": args.workload, "blocks": 30, "hidden": 3072, "heads": 24, "ffn": 12288,
                       "tokens": cfg.tokens, "abits": abits, "rht": rotate, "replicas": world,
                       "launch": "one CUDA graph per step",
                       "weights": args.weights,
                       "l2": "%s GB of weights streamed per step (> 126 MB L2)" % ("3.4" if args.weights == "prepacked" else "1.7")},
            "gpu_launches": 240 * args.steps,
            "linear_tops": linear_ops / (ms * 1e-3) / 1e12,
            "e2e": {"value": e2e_ms, "unit": "ms", "h2d_bytes_per_step": x_host.numel() * 2,
                    "d2h_bytes_per_step": out_host.numel() * 2},
            "clocks": clocks,
            "parity": {"tolerance": 1e-2, "linear_rel_fro_max": parity["output"]["linear_max"],
                       "linear_rel_fro_per_block": [round(v, 6) for v in parity["linear"]],
                       "teacher_forced_rel_fro_max": parity["output"]["teacher_forced_max"],
                       "free_running_rel_fro_output": parity["output"]["free_running"],
                       "code_mismatch_fraction_max": parity["output"]["code_mismatch_max"],
                       "teacher_forced_rel_fro_per_block": [round(v, 6) for v in parity["teacher_forced"]],
                       "free_running_rel_fro_per_block": [round(v, 6) for v in parity["free_running"]],
                       "code_mismatch_fraction_per_block": [round(v, 8) for v in parity["code_mismatch"]]}}), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=200)
    parser.add_argument("--warmup", type=int, default=10)
    parser.add_argument("--workload", default="c2", choices=sorted(WORKLOADS) + sorted(DIT_WORKLOADS) +
                        ["nsplit_ffn_up", "c5_sweep", "m4096_ffn_up_channel"])
    parser.add_argument("--impl", default="b200", choices=["b200", "reference"])
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--chunks", type=int, default=4, help="nsplit_ffn_up: token chunks of the gather / GEMM overlap")
    parser.add_argument("--weights", default="packed", choices=["packed", "prepacked"],
                        help="packed: the checkpoint format (two int4 per byte), unpacked in shared memory by the "
                             "kernel; prepacked: an int8 copy made once at load time (sq_prepack_weights), twice the "
                             "weight bytes, reported as a labelled variant")
    args = parser.parse_args()
    if args.workload == "nsplit_ffn_up":
        if args.steps == 200:
            args.steps = 50
        run_nsplit(args)
        return
    if args.workload in ("c5_sweep", "m4096_ffn_up_channel"):
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device: the B200 path has no CPU fallback.")
        if args.steps == 200:
            args.steps = 20
        (run_sweep if args.workload == "c5_sweep" else run_channel)(args)
        return
    if args.workload in DIT_WORKLOADS:
        if args.steps == 200:
            args.steps = 20
        run_dit(args)
        return
    m, k, n, abits, rotate = WORKLOADS[args.workload]

    if args.impl == "reference":
        run_reference(args, m, k, n, abits, rotate)
        return

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    distributed = world > 1
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the B200 path has no CPU fallback.")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if distributed:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)

    import __graft_entry__ as entry
    entry.load_package()
    from fastwamjoint_quantization_b200 import native

    oracle = load_oracle()
    # rank r of a sharded job holds rows [r*M, (r+1)*M) of a global batch of world*M tokens: same
    # weights (seed 0), its own activations (x seed = rank)
    case = oracle.prepare_token_linear(m, k, n, abits=abits, seed=0, x_seed=None if world == 1 else 1000 + rank)
    packed_host = oracle.pack_signed_int4(case["qweight"])
    signs = None if case["signs"] is None else case["signs"].to(device)

    # rotating input sets so every step reads x and W from HBM, not from L2
    set_bytes = algorithmic_bytes(m, k, n, rotate)
    nsets = max(2, -(-2 * L2_BYTES // set_bytes))
    xs, packs, wss = [], [], []
    for i in range(nsets):
        xs.append((case["x"].float() * (1.0 + 0.001 * i)).to(torch.bfloat16).to(device))
        packs.append(native.prepack_weights(packed_host.to(device)) if args.weights == "prepacked"
                     else packed_host.to(device).clone())
        wss.append(case["weight_scales"].to(device).clone())
    bias = case["bias"].to(device)

    lib_ws = native._lib.load_library().sq_workspace_bytes(m, k) + native._lib.load_library().sq_split_workspace_bytes(m)
    outs = [torch.empty((m, n), device=device, dtype=torch.bfloat16) for _ in range(nsets)]
    workspace = torch.empty((lib_ws,), device=device, dtype=torch.uint8)

    def step(i):
        j = i % nsets
        return native.linear(xs[j], packs[j], wss[j], bias, abits=abits, mode="token", signs=signs, out=outs[j],
                             workspace=workspace)

    def barrier():
        if distributed:
            dist.barrier()
        torch.cuda.synchronize()

    def graph_of(fn, count):
        """Capture `count` calls of fn(i) into one CUDA graph (launch cost leaves the timed region, as in
        the deployed path, where a whole denoising step is one graph)."""
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            fn(0)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(count):
                fn(i)
        return graph

    def timed_replay(graph):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        graph.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1)

    # correctness of what is being timed (small slice, against the oracle)
    out0 = step(0)
    rows = min(m, 64)
    want = oracle.linear_token(case["x"][:rows], case["qweight"], case["weight_scales"], case["bias"], abits=abits,
                               signs=case["signs"], want_accumulators=False)["out"]
    err = ((out0[:rows].cpu().float() - want.float()).norm() / want.float().norm()).item()
    if not err < 1e-2:
        raise SystemExit(f"bench output differs from the oracle: relative Frobenius error {err}")

    warmup = max(args.warmup, 3)
    for i in range(warmup):
        step(i)
    step_graph = graph_of(step, args.steps)
    step_graph.replay()  # one untimed replay of the whole graph
    torch.cuda.synchronize()

    def timed_replays(graph, count):
        """`count` replays of a K-step graph, each bracketed by its own CUDA events on the launching stream."""
        pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(count)]
        for e0, e1 in pairs:
            e0.record()
            graph.replay()
            e1.record()
        torch.cuda.synchronize()
        return sorted(e0.elapsed_time(e1) for e0, e1 in pairs)

    # Timed region: at least 30 replays of the K-step graph and at least 50 ms of GPU time in total, so the clock
    # samplers (100 ms period here, the driver's outside) see the GPU under this load; the median replay is the
    # reported K steps, the best one is given next to it.
    probe_ms = timed_replay(step_graph)
    replays = max(30, int(50.0 / max(probe_ms, 1e-3)) + 1)
    sampler = ClockSampler(local_rank)
    sampler.start()
    barrier()
    replay_ms = timed_replays(step_graph, replays)
    barrier()
    elapsed_ms = replay_ms[len(replay_ms) // 2]
    best_ms = replay_ms[0]

    # Sustained: the same graph back to back for two seconds, clocks sampled meanwhile (a burst of a millisecond
    # runs at the boost clock; a long load settles at the power-capped clock)
    sustained_sampler = ClockSampler(local_rank)
    s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sustained_replays = max(1, int(2000.0 / max(elapsed_ms, 1e-3)))
    sustained_sampler.start()
    s0.record()
    for _ in range(sustained_replays):
        step_graph.replay()
    s1.record()
    torch.cuda.synchronize()
    sustained_clocks = sustained_sampler.stop()
    sustained_ms_per_step = s0.elapsed_time(s1) / (sustained_replays * args.steps)

    # the two kernels alone, same rotation of inputs, for the roofline
    pre = [native.prepass(xs[j], abits=abits, mode="token", signs=signs) for j in range(nsets)]

    def gemm_only(i):
        j = i % nsets
        native.gemm(pre[j][0], packs[j], wss[j], pre[j][1], bias, out_dtype=torch.bfloat16, out=outs[j],
                    int4_range=abits == 4)  # what sq_linear passes for the codes of a 4-bit pre-pass

    def prepass_only(i):
        j = i % nsets
        native.prepass(xs[j], abits=abits, mode="token", signs=signs, out=pre[j])

    gemm_graph = graph_of(gemm_only, args.steps)
    timed_replay(gemm_graph)
    gemm_ms = timed_replays(gemm_graph, max(10, replays // 3))
    gemm_ms = gemm_ms[len(gemm_ms) // 2] / args.steps
    prepass_graph = graph_of(prepass_only, args.steps)
    timed_replay(prepass_graph)
    prepass_ms = timed_replays(prepass_graph, max(10, replays // 3))
    prepass_ms = prepass_ms[len(prepass_ms) // 2] / args.steps

    # End to end through the public call with HOST buffers: every step copies its input from pinned host memory
    # and its result back to pinned host memory.  Copies and compute of consecutive steps overlap on three
    # streams with two device buffers each way (the copy engines are independent of the SMs); every byte of
    # every step still crosses PCIe inside the timed region.
    depth = 2
    x_host = [case["x"].pin_memory() for _ in range(depth)]
    out_host = [torch.empty((m, n), dtype=torch.bfloat16).pin_memory() for _ in range(depth)]
    x_dev = [torch.empty_like(xs[0]) for _ in range(depth)]
    out_dev = [torch.empty((m, n), device=device, dtype=torch.bfloat16) for _ in range(depth)]
    ws_dev = [torch.empty((lib_ws,), device=device, dtype=torch.uint8) for _ in range(depth)]
    copy_in, copy_out, main = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.current_stream()
    in_done = [torch.cuda.Event() for _ in range(depth)]
    run_done = [torch.cuda.Event() for _ in range(depth)]
    out_done = [torch.cuda.Event() for _ in range(depth)]

    def e2e_loop(count):
        for i in range(count):
            b, j = i % depth, i % nsets
            with torch.cuda.stream(copy_in):
                copy_in.wait_event(run_done[b])  # the previous use of this input buffer has been consumed
                x_dev[b].copy_(x_host[b], non_blocking=True)
                in_done[b].record()
            main.wait_event(in_done[b])
            main.wait_event(out_done[b])  # the previous result in this output buffer has left the device
            native.linear(x_dev[b], packs[j], wss[j], bias, abits=abits, mode="token", signs=signs, out=out_dev[b],
                          workspace=ws_dev[b])
            run_done[b].record()
            with torch.cuda.stream(copy_out):
                copy_out.wait_event(run_done[b])
                out_host[b].copy_(out_dev[b], non_blocking=True)
                out_done[b].record()
        main.wait_stream(copy_in)
        main.wait_stream(copy_out)

    e2e_steps = max(5, min(args.steps, 100))
    e2e_loop(4)
    barrier()
    h0, h1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    h0.record()
    e2e_loop(e2e_steps)
    h1.record()
    barrier()
    e2e_ms = h0.elapsed_time(h1)

    # what the host link alone allows: the same two copies per step on the same streams and buffers, no kernel
    def copies_only(count):
        for i in range(count):
            b = i % depth
            with torch.cuda.stream(copy_in):
                x_dev[b].copy_(x_host[b], non_blocking=True)
            with torch.cuda.stream(copy_out):
                out_host[b].copy_(out_dev[b], non_blocking=True)
        main.wait_stream(copy_in)
        main.wait_stream(copy_out)

    copies_only(4)
    barrier()
    c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    c0.record()
    copies_only(e2e_steps)
    c1.record()
    barrier()
    copy_ms = c0.elapsed_time(c1)
    e2e_err = ((out_host[0][:rows].float() - want.float()).norm() / want.float().norm()).item()
    if not e2e_err < 1e-2:
        raise SystemExit(f"end-to-end output differs from the oracle: relative Frobenius error {e2e_err}")
    clocks = sampler.stop()
    status = native.device_status()
    if status != 0:
        raise SystemExit(f"a kernel gave up a bounded wait: device status {status}")

    if distributed:
        t = torch.tensor([elapsed_ms, e2e_ms, copy_ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms, e2e_ms, copy_ms = t.tolist()

    ops_per_step = 2.0 * m * n * k
    tops = world * ops_per_step * args.steps / (elapsed_ms * 1e-3) / 1e12
    e2e_tops = world * ops_per_step * e2e_steps / (e2e_ms * 1e-3) / 1e12

    if rank == 0:
        peaks = {}
        peaks_file = ROOT / "MEASURED_PEAKS.json"
        if peaks_file.exists():
            peaks = json.loads(peaks_file.read_text())
        hbm_peak = float(peaks.get("hbm_gbs", 6650.0))
        try:
            int8_peak = measure_int8_peak(device)
            int8_source = "torch._int_mm 8192^3 best of 10, measured in this run (int8 is not in MEASURED_PEAKS.json)"
        except Exception as exc:  # keep the bench line; say where the denominator came from
            int8_peak = 2.0 * float(peaks.get("bf16_tflops", 1590.0))
            int8_source = "2 x measured bf16 peak (torch._int_mm failed: %s)" % type(exc).__name__
        gemm_tops = ops_per_step / (gemm_ms * 1e-3) / 1e12
        t_compute = ops_per_step / (int8_peak * 1e12)
        t_hbm = algorithmic_bytes(m, k, n, rotate) / (hbm_peak * 1e9)
        fixed_int8_peak = 2.0 * float(peaks.get("bf16_tflops", 1590.0))  # a run-independent denominator
        if t_compute >= t_hbm:
            # `traffic` (DRAM bytes per launch) is not measured in this run: the ncu summary under profiles/ named
            # for this kernel and workload holds it
            roofline = {"bound": "tensor", "achieved": gemm_tops, "peak": int8_peak, "unit": "TOP/s",
                        "frac": gemm_tops / int8_peak, "traffic": None, "peak_source": int8_source,
                        "frac_of_2x_measured_bf16": gemm_tops / fixed_int8_peak,
                        "peak_2x_measured_bf16": fixed_int8_peak}
        else:
            gbs = algorithmic_bytes(m, k, n, rotate) / (gemm_ms * 1e-3) / 1e9
            roofline = {"bound": "hbm", "achieved": gbs, "peak": hbm_peak, "unit": "GB/s", "frac": gbs / hbm_peak,
                        "traffic": None, "peak_source": "MEASURED_PEAKS.json" if peaks else "fallback"}
        roofline["kernel"] = "sq_gemm_tc_kernel"
        roofline["weights"] = args.weights
        roofline["gemm_ms"] = gemm_ms
        roofline["prepass_ms"] = prepass_ms
        roofline["prepass_gbs"] = (2 * m * k + m * k + 4 * m) / (prepass_ms * 1e-3) / 1e9
        roofline["prepass_frac_of_hbm"] = roofline["prepass_gbs"] / hbm_peak
        roofline["whole_linear_frac"] = max(t_compute, t_hbm) / (elapsed_ms / args.steps * 1e-3)
        line = {
            "metric": "W4A%d%s GEMM int-TOPS" % (abits, "+RHT" if rotate else ""), "value": tops, "unit": "TOPS",
            "n_gpus": world, "steps": args.steps, "warmup": warmup,
            "ms_per_step": elapsed_ms / args.steps, "ms_per_step_best": best_ms / args.steps, "replays": replays,
            "timed_region_ms": sum(replay_ms),
            "sustained": {"seconds": sustained_replays * args.steps * sustained_ms_per_step / 1e3,
                          "ms_per_step": sustained_ms_per_step,
                          "tops": world * ops_per_step / (sustained_ms_per_step * 1e-3) / 1e12,
                          "sm_mhz": sustained_clocks["sm_mhz"], "reasons": sustained_clocks["reasons"]},
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "int8 x int4 -> int32", "data": "synthetic",
            "config": {"workload": args.workload, "M_per_gpu": m, "K": k, "N": n, "abits": abits, "rht": rotate,
                       "weight_scales": "fp16 group-128", "activation_scales": "per-token",
                       "weights": ("int8 copy made once at load from the packed int4 format (variant, twice the weight bytes)"
                                   if args.weights == "prepacked" else "packed int4 (checkpoint format), unpacked in shared memory"),
                       "sharding": "tokens (M) across ranks, weights replicated, no collective",
                       "l2": "rotating %d input sets (%.0f MB > 126 MB L2)" % (nsets, nsets * set_bytes / 1e6),
                       "launch": "the K steps are one CUDA graph; value = median of `replays` replays"},
            "gpu_launches": 2 * args.steps * replays,
            "e2e": {"value": e2e_tops, "unit": "TOPS", "h2d_bytes_per_step": x_host[0].numel() * 2,
                    "d2h_bytes_per_step": out_host[0].numel() * 2, "ms_per_step": e2e_ms / e2e_steps,
                    "pipeline": "host->device copy, linear and device->host copy of consecutive steps overlap (3 streams, 2 buffers)",
                    "copies_only_ms_per_step": copy_ms / e2e_steps,
                    "host_link_gbs_each_way": x_host[0].numel() * 2 / (copy_ms / e2e_steps * 1e-3) / 1e9,
                    "frac_of_host_link_ceiling": copy_ms / e2e_ms},
            "roofline": roofline, "clocks": clocks, "parity_rel_fro": err,
        }
        if not args.no_cpu_baseline and world == 1:  # reported at N = 1 only: the other ranks would share the cores
            cores = os.cpu_count() or 1
            torch.set_num_threads(cores)
            median, repeats = time_cpu(cpu_forward_factory(oracle, case))
            line["cpu_baseline"] = {"value": ops_per_step / median / 1e12, "unit": "TOPS", "cores": cores, "kind": "port",
                                    "sample": "median of %d full passes of the workload" % repeats}
        print(json.dumps(line), flush=True)
    if distributed:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
