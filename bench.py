"""Benchmark of the W4A16 decode path (the configuration the headline metric is quoted on).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (BASELINE.json configs[1]): the four Llama-3-8B-shaped AWQ int4 linears
(K x N: qkv 4096x6144, o 4096x4096, gate_up 4096x28672, down 14336x4096; group 128, bf16
activations ~N(0,1), int4 weights and zero points uniform in 0..15, bf16 scales
|N(0,1)|*0.01+1e-3) at M in {1, 4, 16, 64}.  One STEP = those 16 GEMMs.  Data are seeded
synthetic tensors of these shapes (no checkpoint is involved).

Metric: weight-stream bandwidth = int4 weight bytes of the GEMMs of a step / time.
* `value`     inputs resident in HBM; the step is replayed as a CUDA graph; weights rotate over
              several full copies of the layer so that no GEMM finds its weights in L2.
* `e2e`       the same GEMMs issued one by one through the operator API with HOST activations
              and outputs: pinned host -> device copy of A and device -> host copy of C inside
              the timed region (weights are model state and stay on the device).
* `roofline`  algorithmic bytes of the GEMM launches in the timed region / their time, against
              the measured HBM copy bandwidth of this machine pool.
* `cpu_baseline`  the reference's CPU formulation (fp32 dequantise, then matmul) on the host
              cores for a bounded sample of the same workload.

With N > 1 (one process per GPU under torchrun) every linear is column-parallel: rank r holds
columns [r N/g, (r+1) N/g) and the output slices are all-gathered over NCCL.  The total work is
the same for every N (strong scaling).
"""

from __future__ import annotations

import argparse
import json
import os
import pathlib
import statistics
import subprocess
import sys
import tempfile
import time

import torch

ROOT = pathlib.Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

SHAPES = (("qkv", 4096, 6144), ("o", 4096, 4096), ("gate_up", 4096, 28672), ("down", 14336, 4096))
MS = (1, 4, 16, 64)
GROUP = 128
SEED = 20260728 + 1000
L2_BYTES = 126 * 1024 * 1024


def weight_bytes(k, n):
    return k * n // 2


def algorithmic_bytes(m, k, n):
    g = k // GROUP
    return k * n // 2 + g * n * 2 + g * n // 2 + m * k * 2 + m * n * 2


def measured_hbm_peak():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.file = index, None, None

    def __enter__(self):
        try:
            self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=self.file, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None
        return self

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()

    def summary(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.file is None:
            return out
        try:
            rows = [r.split(",") for r in pathlib.Path(self.file.name).read_text().strip().splitlines() if r.strip()]
            os.unlink(self.file.name)
            clocks = [float(r[0]) for r in rows]
            if clocks:
                # the median over the busy part: drop samples at idle clocks
                busy = [c for c in clocks if c > 0.5 * max(clocks)] or clocks
                out["sm_mhz"] = statistics.median(busy)
                out["sm_max_mhz"] = float(rows[0][1])
            names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
            for i, name in enumerate(names):
                if any(r[2 + i].strip().lower().startswith("active") for r in rows):
                    out["reasons"].append(name)
            out["samples"] = len(rows)
        except Exception:
            pass
        return out


# ---------------------------------------------------------------------------------------------------
def make_layer(rank, world, device, copy_index):
    """One copy of the four linears, column shard `rank` of `world`, prepared through the
    library's own AWQ -> Marlin repack."""
    from infiniops_b200 import capi

    layer = {}
    for si, (name, k, n) in enumerate(SHAPES):
        n_local = n // world
        gen = torch.Generator(device=device).manual_seed(SEED + si + 100 * copy_index + 10000 * rank)
        awq = torch.randint(-2**31, 2**31 - 1, (k, n_local // 8), dtype=torch.int32, device=device, generator=gen)
        marlin = torch.empty((k // 16, 2 * n_local), dtype=torch.int32, device=device)
        capi.awq_marlin_repack(awq, k, n_local, 4, False, marlin)
        scales = (torch.randn((k // GROUP, n_local), device=device, generator=gen).abs() * 0.01 + 1e-3).bfloat16()
        zeros = torch.randint(-2**31, 2**31 - 1, (k // GROUP, n_local // 8), dtype=torch.int32, device=device,
                              generator=gen)
        layer[name] = {"awq": awq if copy_index == 0 else None, "marlin": marlin, "scales": scales, "zeros": zeros,
                       "k": k, "n": n_local}
    return layer


def run_ours(args):
    import torch.distributed as dist

    from infiniops_b200 import capi, parallel

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"

    layer_bytes = sum(weight_bytes(k, n) for _, k, n in SHAPES) // world
    # Rotate through >= 3x L2 of weights; a multiple of len(MS) so that the j-th M of a step always
    # takes copy 4 * phase + j and a (linear, copy) pair returns only after all copies were streamed.
    copies = len(MS) * max(1, -(-3 * L2_BYTES // (layer_bytes * len(MS))))
    layers = [make_layer(rank, world, device, c) for c in range(copies)]
    acts = {(name, m): torch.randn((m, k), device=device, generator=torch.Generator(device=device).manual_seed(
        SEED + 7 * m + i)).bfloat16() for i, (name, k, _) in enumerate(SHAPES) for m in MS}
    # The 16 output slices live in one arena, so that the slices of a whole step can also be exchanged
    # with a single all-gather (--gather step); each slice starts on a 16-byte boundary.
    arena_elems = sum(-(-(m * (n // world)) // 8) * 8 for _, _, n in SHAPES for m in MS)
    arena = torch.empty(arena_elems, dtype=torch.bfloat16, device=device)
    arena_all = torch.empty((world, arena_elems), dtype=torch.bfloat16, device=device) if world > 1 else None
    outs, off = {}, 0
    for name, _, n in SHAPES:
        for m in MS:
            outs[(name, m)] = arena[off:off + m * (n // world)].view(m, n // world)
            off += -(-(m * (n // world)) // 8) * 8
    gathered = {(name, m): torch.empty((world, m, n // world), dtype=torch.bfloat16, device=device)
                for name, _, n in SHAPES for m in MS} if world > 1 else None
    need = max(capi.lib().infiniops_b200_marlin_gemm_scratch_bytes(m, n // world, k) for _, k, n in SHAPES for m in MS)
    scratch = torch.zeros(need, dtype=torch.uint8, device=device)

    phases = copies // len(MS)

    if args.gather == "auto":
        args.gather = "step"
    comm = None
    if world > 1 and args.gather not in ("serial", "step"):
        comm = torch.cuda.Stream(priority=-1) if args.gather == "overlap-prio" else torch.cuda.Stream()

    def step(phase, stream=None):
        """The 16 GEMMs back to back on the compute stream; with N > 1 every all-gather runs on a second
        stream behind its GEMM, so the exchange of one linear overlaps the GEMM of the next."""
        launches = 0
        main = torch.cuda.current_stream()
        for mi, m in enumerate(MS):
            for name, k, n in SHAPES:
                w = layers[phase * len(MS) + mi][name]
                capi.marlin_gemm(acts[(name, m)], w["marlin"], None, w["scales"], w["zeros"], capi.QTYPE_UINT4, m,
                                 w["n"], k, outs[(name, m)], stream=stream, scratch_buf=scratch)
                launches += 1
                if world > 1 and args.gather != "step":
                    if comm is None:
                        parallel.gather_columns(outs[(name, m)], gathered[(name, m)])
                    else:
                        comm.wait_stream(main)
                        with torch.cuda.stream(comm):
                            parallel.gather_columns(outs[(name, m)], gathered[(name, m)])
        if comm is not None:
            main.wait_stream(comm)
        if world > 1 and args.gather == "step":
            dist.all_gather_into_tensor(arena_all.view(-1), arena)  # [g, arena]: rank-major copies of every slice
        return launches

    # warm-up outside any graph (function attributes, tensor maps, NCCL channels)
    for phase in range(phases):
        step(phase)
    torch.cuda.synchronize()
    assert capi.scratch_status(scratch) == 0, f"a GEMM kernel gave up on a wait: {scratch[:192].view(torch.int32).tolist()}"

    # The step as CUDA graphs, one per weight copy rotation, so replays keep rotating the weights.
    graphs = []
    launches_per_step = 0
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    n_graphs = phases
    with torch.cuda.stream(side):
        for phase in range(n_graphs):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                launches_per_step = step(phase, stream=side.cuda_stream)
            graphs.append(g)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(max(args.warmup, 3)):
        graphs[i % n_graphs].replay()
    barrier()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as clocks:
        time.sleep(0.15)
        barrier()
        start.record()
        for i in range(args.steps):
            graphs[i % n_graphs].replay()
        stop.record()
        barrier()
        time.sleep(0.15)
    elapsed_ms = start.elapsed_time(stop)
    assert capi.scratch_status(scratch) == 0, f"a GEMM kernel gave up on a wait: {scratch[:192].view(torch.int32).tolist()}"

    # ---- end to end through the operator call with host buffers -------------------------------
    host_in = {key: t.cpu().pin_memory() for key, t in acts.items()}
    full_n = {name: n for name, _, n in SHAPES}
    host_out = {key: torch.empty((key[1], full_n[key[0]]), dtype=torch.bfloat16).pin_memory() for key in acts}
    dev_in = {key: torch.empty_like(t) for key, t in acts.items()}
    h2d = sum(t.numel() * 2 for t in host_in.values())
    d2h = sum(t.numel() * 2 for t in host_out.values())

    def e2e_step(phase):
        for mi, m in enumerate(MS):
            for name, k, n in SHAPES:
                w = layers[phase * len(MS) + mi][name]
                dev_in[(name, m)].copy_(host_in[(name, m)], non_blocking=True)
                capi.marlin_gemm(dev_in[(name, m)], w["marlin"], None, w["scales"], w["zeros"], capi.QTYPE_UINT4, m,
                                 w["n"], k, outs[(name, m)], scratch_buf=scratch)
                if world > 1:
                    parallel.gather_columns(outs[(name, m)], gathered[(name, m)])
                    full = gathered[(name, m)].permute(1, 0, 2).reshape(m, n)
                    host_out[(name, m)].copy_(full, non_blocking=True)
                else:
                    host_out[(name, m)].copy_(outs[(name, m)], non_blocking=True)

    for i in range(3):
        e2e_step(i % phases)
    barrier()
    e2e_steps = max(3, min(args.steps, 50))
    e_start, e_stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e_start.record()
    for i in range(e2e_steps):
        e2e_step(i % phases)
    e_stop.record()
    barrier()
    e2e_ms = e_start.elapsed_time(e_stop)

    times = torch.tensor([elapsed_ms, e2e_ms], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    elapsed_ms, e2e_ms = (float(v) for v in times.cpu())

    step_weight_bytes = sum(weight_bytes(k, n) for _, k, n in SHAPES) * len(MS)
    step_algo_bytes = sum(algorithmic_bytes(m, k, n // world) for _, k, n in SHAPES for m in MS)  # per GPU
    ms_per_step = elapsed_ms / args.steps
    value = step_weight_bytes / (ms_per_step * 1e-3) / 1e9
    e2e_value = step_weight_bytes / (e2e_ms / e2e_steps * 1e-3) / 1e9
    peak, peak_kind = measured_hbm_peak()
    achieved = step_algo_bytes / (ms_per_step * 1e-3) / 1e9

    result = {
        "metric": "W4A16 GEMM weight HBM GB/s (decode)", "value": value, "unit": "GB/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "configs[1]: Llama-3-8B-shaped AWQ W4A16 linears (qkv, o, gate_up, down), g=128, "
                               "M in {1,4,16,64}; one step = these 16 GEMMs",
                   "parallelism": "single GPU" if world == 1 else
                   f"column-parallel N-shard x{world} + " + ("one NCCL all-gather per step over the 16 output slices"
                                                               if args.gather == "step" else
                                                               f"NCCL all-gather per linear ({args.gather})"),
                   "l2": f"inputs larger than L2: {copies} full weight copies "
                         f"({copies * layer_bytes / 1e6:.0f} MB per GPU) used in rotation",
                   "launch": "CUDA graph replay of the step"},
        "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "steps": e2e_steps, "note": "host activations in, host outputs out, one operator call per GEMM"},
        "gpu_launches": launches_per_step * args.steps,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "peak_kind": f"of {peak_kind}", "traffic": TRAFFIC_BYTES_PER_STEP if world == 1 else None,
                     "traffic_unit": "DRAM bytes per step (16 launches), scaled from one ncu capture",
                     "kernel": "W4A16GemmKernel", "algorithmic_bytes_per_step": step_algo_bytes},
        "clocks": clocks.summary(),
    }
    if rank == 0:
        if world == 1 and not args.no_cpu_baseline:
            result["cpu_baseline"] = cpu_baseline(layers[0], sample_ms=MS, repeats=12)
        print(json.dumps(result), flush=True)
    if world > 1:
        _shutdown(dist, graphs)


# DRAM bytes (read + write) of the 16 GEMM launches of one step.  From the ncu capture of the
# M=16, K=4096, N=28672 launch (profiles/w4a16_gemm_decode_m16_k4096_n28672.md): 61.84 MB measured
# against 62.06 MB algorithmic, ratio 0.996; the other launches stream their weights once in the same
# way, so the step's traffic is taken as its algorithmic bytes times that ratio (single GPU).
TRAFFIC_BYTES_PER_STEP = int(465084416 * 61.84 / 62.06)


# ---------------------------------------------------------------------------------------------------
def cpu_reference_problem(layer):
    """Unpacks the device weights of one layer copy into what the CPU formulation consumes."""
    from oracle import quant as oq

    problem = {}
    for name, k, _ in SHAPES:
        w = layer[name]
        q = oq.awq_unpack(w["awq"].cpu().numpy(), 4)
        zeros_packed = w["zeros"].cpu().numpy().view("uint32")
        zeros = torch.from_numpy(
            ((zeros_packed[:, :, None] >> (4 * torch.arange(8).numpy().astype("uint32"))[None, None, :]) & 0xF)
            .reshape(zeros_packed.shape[0], -1).astype("float32"))
        problem[name] = (torch.from_numpy(q.astype("float32")), w["scales"].float().cpu(), zeros, k, w["n"])
    return problem


def cpu_pass(problem, ms):
    """fp32 dequantise + matmul for every linear at every M in `ms` (the reference's CPU path,
    tests/test_moe_wna16_gemm.py:397-404,437 of the reference)."""
    out = None
    for m in ms:
        for name, _, _ in SHAPES:
            q, scales, zeros, k, n = problem[name]
            a = torch.randn((m, k)).bfloat16()
            w = (q - zeros.repeat_interleave(GROUP, dim=0)) * scales.repeat_interleave(GROUP, dim=0)
            out = a.float() @ w
    return out


def cpu_baseline(layer, sample_ms, repeats):
    torch.set_num_threads(os.cpu_count() or 1)
    problem = cpu_reference_problem(layer)
    best = float("inf")
    for _ in range(repeats):
        t0 = time.perf_counter()
        cpu_pass(problem, sample_ms)
        best = min(best, time.perf_counter() - t0)
    nbytes = sum(weight_bytes(k, n) for _, (_, _, _, k, n) in problem.items()) * len(sample_ms)
    return {"value": nbytes / best / 1e9, "unit": "GB/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"the four linears at M in {list(sample_ms)}, best of {repeats} passes "
                      f"({best:.2f} s per pass, {best * repeats:.0f} s of CPU work)"}


def run_reference(args):
    """The reference's own CPU implementation of the path (the oracle port of its dequantise-
    then-matmul formulation), all host threads, same config and metric."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    torch.set_num_threads(os.cpu_count() or 1)
    gen_layer = {}
    from oracle import quant as oq

    for si, (name, k, n) in enumerate(SHAPES):
        gen = torch.Generator().manual_seed(SEED + si)
        awq = torch.randint(-2**31, 2**31 - 1, (k, n // 8), dtype=torch.int32, generator=gen)
        scales = (torch.randn((k // GROUP, n), generator=gen).abs() * 0.01 + 1e-3).bfloat16()
        zeros = torch.randint(-2**31, 2**31 - 1, (k // GROUP, n // 8), dtype=torch.int32, generator=gen)
        gen_layer[name] = {"awq": awq, "scales": scales, "zeros": zeros, "n": n}
    problem = cpu_reference_problem(gen_layer)
    sample = (16,)
    for _ in range(min(args.warmup, 1)):
        cpu_pass(problem, sample)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_pass(problem, sample)
    elapsed = time.perf_counter() - t0
    nbytes = sum(weight_bytes(k, n) for _, k, n in SHAPES) * len(sample)
    value = nbytes * args.steps / elapsed / 1e9
    cores = torch.get_num_threads()
    print(json.dumps({
        "impl": "reference", "metric": "W4A16 GEMM weight HBM GB/s (decode)", "value": value, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": min(args.warmup, 1), "ms_per_step": elapsed / args.steps * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "configs[1]: Llama-3-8B-shaped AWQ W4A16 linears (qkv, o, gate_up, down), g=128; "
                               "each step = the four linears at M=16 (bounded sample of the 16-GEMM step)"},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": cores, "kind": "port",
                         "sample": "four linears at M=16 per step, fp32 dequantise + torch matmul on the host"},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


def run_moe(args):
    """Mixtral-8x7B-shaped MoE layer (BASELINE.json configs[3]): E=8, top-2, hidden 4096, intermediate 14336,
    GPTQ-symmetric int4 g=128, bf16; router topk_softmax -> moe_align_block_size(64) -> w13 GEMM -> silu_and_mul
    -> w2 GEMM -> moe_sum.  Metric: tokens/s of the whole layer for `--tokens` tokens (global).  With N > 1 the
    experts are split over the ranks and the tokens are data-parallel (T/N each) with all-to-all dispatch and
    combine (strong scaling: the same global batch for every N)."""
    import torch.distributed as dist

    from infiniops_b200 import capi, moe_layer, parallel

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    experts, top_k, hidden, inter, block = 8, 2, 4096, 14336, 64
    e_local = experts // world
    t_local = max(1, args.tokens // world)
    gen = torch.Generator(device=dev).manual_seed(SEED + 3000 + rank)

    def packed(k, n):
        out = torch.empty((e_local, k // 16, 2 * n), dtype=torch.int32, device=dev)
        for e in range(e_local):
            src = torch.randint(-2**31, 2**31 - 1, (k // 8, n), dtype=torch.int32, device=dev, generator=gen)
            capi.gptq_marlin_repack(src, None, k, n, 4, False, out[e])
        scales = (torch.randn((e_local, k // GROUP, n), device=dev, generator=gen).abs() * 0.01 + 1e-3).bfloat16()
        return out, scales

    w13, s13 = packed(hidden, 2 * inter)
    w2, s2 = packed(inter, hidden)
    runner = moe_layer.RoutedExperts(moe_layer.ExpertWeights(w13, s13, None, w2, s2, None, hidden, inter), block)
    x = torch.randn((t_local, hidden), device=dev, generator=gen).bfloat16()
    logits = torch.randn((t_local, experts), device=dev, generator=gen)
    launches = [0]

    def step():
        weights, ids = moe_layer.route_softmax(logits, top_k)
        if world == 1:
            launches[0] = 8   # router, sort, 2 x (gather + GEMM), silu_and_mul, moe_sum
            return moe_layer.single_gpu_layer(x, weights, ids, runner)
        launches[0] = 9
        return parallel.expert_parallel_layer(
            x, ids, weights, experts, top_k, runner,
            lambda routed: _moe_sum(capi, routed))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    steps = min(args.steps, 50)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as clocks:
        barrier()
        e0.record()
        for _ in range(steps):
            out = step()
        e1.record()
        barrier()
    ms = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms_per_step = float(ms) / steps
    assert capi.scratch_status(capi.scratch(dev, 0)) == 0
    tokens = t_local * world
    flops = tokens * top_k * (2 * hidden * 2 * inter + 2 * inter * hidden)
    if rank == 0:
        print(json.dumps({
            "metric": "MoE tokens/s", "value": tokens / (ms_per_step * 1e-3), "unit": "tokens/s", "n_gpus": world,
            "steps": steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"configs[3]: Mixtral-8x7B-shaped MoE layer, E=8 top-2 H=4096 I=14336, T={tokens}",
                       "parallelism": "single GPU" if world == 1 else f"expert-parallel x{world}, NCCL all-to-all",
                       "l2": "inputs larger than L2: 705 MB of expert weights per layer pass"},
            "tflops": flops / (ms_per_step * 1e-3) / 1e12, "gpu_launches": launches[0] * steps,
            "clocks": clocks.summary()}), flush=True)
    if world > 1:
        _shutdown(dist)


def _shutdown(dist, graphs=None):
    """Releases captured graphs (they hold NCCL kernels) before the process group goes away; a
    watchdog ends the process if the teardown itself blocks -- the result line is already out."""
    import gc
    import threading

    threading.Thread(target=lambda: (time.sleep(20), os._exit(0)), daemon=True).start()
    if graphs is not None:
        graphs.clear()
    gc.collect()
    torch.cuda.synchronize()
    dist.barrier()
    dist.destroy_process_group()


def _moe_sum(capi, routed):
    out = torch.empty((routed.shape[0], routed.shape[2]), dtype=routed.dtype, device=routed.device)
    capi.moe_sum(routed, out)
    return out


def run_one(args):
    """One dense AWQ bf16 GEMM `M,K,N`, launched a few times with an L2 flush in between: the small,
    self-terminating case used for profiler captures (`ncu ... python bench.py --one 16,4096,28672`)."""
    from infiniops_b200 import capi

    m, k, n = (int(v) for v in args.one.split(","))
    dev = torch.device("cuda", 0)
    gen = torch.Generator(device=dev).manual_seed(SEED)
    awq = torch.randint(-2**31, 2**31 - 1, (k, n // 8), dtype=torch.int32, device=dev, generator=gen)
    marlin = torch.empty((k // 16, 2 * n), dtype=torch.int32, device=dev)
    capi.awq_marlin_repack(awq, k, n, 4, False, marlin)
    scales = (torch.randn((k // GROUP, n), device=dev, generator=gen).abs() * 0.01 + 1e-3).bfloat16()
    zeros = torch.randint(-2**31, 2**31 - 1, (k // GROUP, n // 8), dtype=torch.int32, device=dev, generator=gen)
    a = torch.randn((m, k), device=dev, generator=gen).bfloat16()
    out = torch.empty((m, n), dtype=torch.bfloat16, device=dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    times = []
    for _ in range(3):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        capi.marlin_gemm(a, marlin, None, scales, zeros, capi.QTYPE_UINT4, m, n, k, out)
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1) * 1e3)
    print(json.dumps({"case": args.one, "us_per_launch_with_launch_gap": times,
                      "algorithmic_bytes": algorithmic_bytes(m, k, n), "flops": 2 * m * k * n}))


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--workload", default="decode", choices=("decode", "moe"),
                        help="decode = the headline W4A16 decode step; moe = Mixtral-shaped MoE layer, tokens/s")
    parser.add_argument("--tokens", type=int, default=1024, help="global tokens of the MoE workload")
    parser.add_argument("--one", default=None, help="M,K,N: run this single GEMM three times (profiling case)")
    parser.add_argument("--gather", default="auto", choices=("auto", "overlap", "overlap-prio", "serial", "step"),
                        help="N > 1, decode: one all-gather per linear on a second stream / a high-priority second "
                             "stream / the compute stream, or one all-gather per step over all 16 output slices; "
                             "auto = step (at 8 ranks a captured all-gather of a few KB costs ~120 us on this pool, "
                             "2.1 ms per step for sixteen of them against 0.33 ms of GEMMs)")
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=200)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", default="ours", choices=("ours", "reference"))
    parser.add_argument("--no-cpu-baseline", action="store_true")
    args = parser.parse_args()
    if args.one:
        run_one(args)
    elif args.workload == "moe" and args.impl == "ours":
        run_moe(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
