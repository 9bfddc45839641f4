"""Benchmark of the W4A16 linear + MoE hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Headline workload (BASELINE.json configs[1]): the four Llama-3-8B-shaped AWQ int4 linears
(K x N: qkv 4096x6144, o 4096x4096, gate_up 4096x28672, down 14336x4096; group 128, bf16
activations ~N(0,1), int4 weights and zero points uniform in 0..15, bf16 scales
|N(0,1)|*0.01+1e-3) at M in {1, 4, 16, 64}.  One STEP = those 16 GEMMs.  Data are seeded
synthetic tensors of these shapes (no checkpoint or dataset is involved).

Metric: weight-stream bandwidth = int4 weight bytes of the GEMMs of a step / time.
* `value`     inputs resident in HBM; the step is the batched dense GEMM (the 16 problems as two
              persistent launches) replayed as a CUDA graph; weights rotate over several full copies of
              the layer so that no GEMM finds its weights in L2.  The timed region of K steps is
              repeated; the median is reported with the spread.
* `e2e`       the same GEMMs issued one by one through the operator API (`infini.ops.marlin_gemm`)
              with HOST activations and outputs: pinned host -> device copy of A and device -> host
              copy of C inside the timed region (weights are model state and stay on the device);
              on one GPU consecutive steps alternate between three sets of buffers and streams.  With
              N > 1: one placed C-ABI GEMM call per GEMM (epilogue peer stores), every rank copying the
              full-width results out; copies and GEMMs on streams of their own.
* `roofline`  algorithmic bytes of the GEMM launches in the timed region / their time, against
              the measured HBM copy bandwidth of this machine pool.
* `cpu_baseline`  the reference's CPU formulation (fp32 dequantise, then matmul) on the host
              cores for a bounded sample of the same workload.
* `per_gemm`, `prefill`, `moe`, `small_kernels`  sub-records, each with its own CUDA-event timing:
              the step as sixteen separate launches; the four linears at M = 4096 (TFLOP/s against the
              measured bf16 peak); the Mixtral- and DeepSeek-shaped MoE layers (tokens/s); repack,
              routers, token sort, silu_and_mul and moe_sum at their layer sizes (GB/s).

With N > 1 (one process per GPU under torchrun) every linear is column-parallel: rank r holds
columns [r N/g, (r+1) N/g) and the GEMM epilogue stores its slice straight into the full-width
result matrix of EVERY rank over NVLink (peer-mapped buffers, plain stores, no multicast); the last
block of a step's last launch raises a flag on each peer and a bounded wait on the flags closes the
step.  No NCCL call is on the decode path.  After the timed region every rank checks that each
gathered slice equals, bit for bit, what that rank's shard computes locally.  The MoE layer is
expert-parallel.  The total work is the same for every N (strong scaling).
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
UINT4B8, UINT4 = 1125899907892224, 1125899906843648
WORKLOAD = ("configs[1]: Llama-3-8B-shaped AWQ W4A16 linears (qkv, o, gate_up, down), g=128, "
            "M in {1,4,16,64}; one step = these 16 GEMMs")
METRIC = "W4A16 GEMM weight HBM GB/s (decode)"


def weight_bytes(k, n):
    return k * n // 2


def algorithmic_bytes(m, k, n, zeros=True):
    g = k // GROUP
    return k * n // 2 + g * n * 2 + (g * n // 2 if zeros else 0) + m * k * 2 + m * n * 2


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            d = json.loads(path.read_text())
            return {"hbm": float(d["hbm_gbs"]), "bf16": float(d["bf16_tflops"]),
                    "bf16_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "kind": "measured"}
        except Exception:
            pass
    return {"hbm": 6650.0, "bf16": 1590.0, "bf16_sustained": 1400.0, "kind": "fallback"}


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


class Dist:
    """Rank bookkeeping (one process per GPU under torchrun; a single process otherwise)."""

    def __init__(self, args):
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(self.local_rank)
        self.device = torch.device("cuda", self.local_rank)
        if self.world > 1:
            import torch.distributed as dist

            dist.init_process_group("nccl", device_id=self.device)
        assert self.world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={self.world}"

    def barrier(self):
        if self.world > 1:
            import torch.distributed as dist

            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(self, values):
        t = torch.tensor(values, dtype=torch.float64, device=self.device)
        if self.world > 1:
            import torch.distributed as dist

            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return [float(v) for v in t.cpu()]

    def all_true(self, flag: bool) -> bool:
        t = torch.tensor([1 if flag else 0], dtype=torch.int32, device=self.device)
        if self.world > 1:
            import torch.distributed as dist

            dist.all_reduce(t, op=dist.ReduceOp.MIN)
        return bool(int(t.cpu()[0]))


def timed_regions(d: Dist, run_steps, steps, repeats):
    """`repeats` timed regions of `steps` steps each, every one bracketed by a barrier and a device
    synchronisation, timed with CUDA events on the launching stream; max over ranks per region.
    Returns the per-region ms-per-step values."""
    out = []
    for _ in range(repeats):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        d.barrier()
        start.record()
        run_steps(steps)
        stop.record()
        d.barrier()
        out.append(d.max_over_ranks([start.elapsed_time(stop)])[0] / steps)
    return out


def spread_of(values):
    med = statistics.median(values)
    return {"median": med, "min": min(values), "max": max(values), "regions": len(values),
            "spread": (max(values) - min(values)) / med if med else None}


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
    from infiniops_b200 import capi

    d = Dist(args)
    world, rank, device = d.world, d.rank, d.device
    peaks = measured_peaks()

    layer_bytes = sum(weight_bytes(k, n) for _, k, n in SHAPES) // world
    # Rotate through >= 3x L2 of weights; a multiple of len(MS) so that the j-th M of a step always
    # takes copy 4 * phase + j and a (linear, copy) pair returns only after all copies were streamed.
    # An even number of phases: the output buffers alternate with the phase (see below).
    phases = max(2, -(-3 * L2_BYTES // (layer_bytes * len(MS))))
    phases += phases % 2
    copies = len(MS) * phases
    layers = [make_layer(rank, world, device, c) for c in range(copies)]
    acts = {(name, m): torch.randn((m, k), device=device, generator=torch.Generator(device=device).manual_seed(
        SEED + 7 * m + i)).bfloat16() for i, (name, k, _) in enumerate(SHAPES) for m in MS}
    keys = [(name, m) for m in MS for name, _, _ in SHAPES]
    full_n = {name: n for name, _, n in SHAPES}
    full_k = {name: k for name, k, _ in SHAPES}

    # Result matrices [M, N] (full width).  With N > 1 they live in an arena every rank maps, in two
    # sets used by alternate steps: a rank that runs one step ahead stores into the other set.
    group = None
    if world > 1:
        from infiniops_b200 import peer

        set_bytes = sum(-(-(m * full_n[name] * 2) // 256) * 256 for name, m in keys)
        prefill_bytes = 0 if args.headline_only else 4096 * max(n for _, _, n in SHAPES) * 2 + 256
        group = peer.PeerGroup(2 * set_bytes + prefill_bytes, device)
        offsets = [{key: group.carve(key[1] * full_n[key[0]] * 2) for key in keys} for _ in range(2)]
        outs = [{key: group.local(offsets[s][key], (key[1], full_n[key[0]]), torch.bfloat16) for key in keys}
                for s in range(2)]
    else:
        outs = [{key: torch.empty((key[1], full_n[key[0]]), dtype=torch.bfloat16, device=device) for key in keys}] * 2
    scratch = torch.zeros(max(capi.lib().infiniops_b200_marlin_gemm_batch_scratch_bytes(),
                              max(capi.lib().infiniops_b200_marlin_gemm_scratch_bytes(m, n // world, k)
                                  for _, k, n in SHAPES for m in MS)), dtype=torch.uint8, device=device)

    # How the slices reach the other ranks: stored by the GEMM epilogue tile by tile ("epilogue"), or by one
    # copy launch behind the GEMMs that sends every slice with whole-warp stores ("broadcast")
    # (measured: the copy launch costs 8 us more per step at N = 2 and 4 us more at N = 4 than it saves, so the
    # epilogue stores are the default at every N)
    gather = "epilogue" if args.gather == "auto" else args.gather

    def problem(phase, key, layer_set=None):
        name, m = key
        w = (layer_set or layers)[phase * len(MS) + MS.index(m)][name]
        peers = ([] if group is None or gather == "broadcast" else
                 [group.address(r, offsets[phase % 2][key]) for r in group.others()])
        return capi.gemm_problem(acts[key], w["marlin"], None, w["scales"], w["zeros"], outs[phase % 2][key], m, w["n"],
                                 w["k"], out_ld=full_n[name], out_col0=rank * w["n"], peer_out=peers)

    tables = [capi.problem_array([problem(phase, key) for key in keys]) for phase in range(phases)]
    # One GPU: the step as two batch calls side by side -- the M = 64 problems on the step's stream, the
    # M <= 16 problems on a second one, each call with its own scratch -- instead of one call whose two
    # launches follow each other: the second call's blocks take the SMs as the first's blocks leave them
    # and so work through the first launch's split-K hand-over instead of waiting for its end.
    side_by_side = group is None and args.decode_streams == 2
    if side_by_side:
        wide = [capi.problem_array([problem(phase, key) for key in keys if key[1] > 32]) for phase in range(phases)]
        narrow = [capi.problem_array([problem(phase, key) for key in keys if key[1] <= 32]) for phase in range(phases)]
        scratch_b = torch.zeros_like(scratch)
        branch = torch.cuda.Stream()
    singles = [[problem(phase, key) for key in keys] for phase in range(phases)]
    signal = None if group is None else group.signal()

    slice_copies = None
    if group is not None and gather == "broadcast":
        def slice_copy(phase, key):
            name, m = key
            n_local = full_n[name] // world
            col_bytes = rank * n_local * 2
            return capi.peer_copy(outs[phase % 2][key].data_ptr() + col_bytes,
                                  [group.address(r, offsets[phase % 2][key]) + col_bytes for r in group.others()],
                                  m, n_local * 2, full_n[name] * 2)
        slice_copies = [(capi.PeerCopy * len(keys))(*[slice_copy(phase, key) for key in keys]) for phase in range(2)]

    def step_batched(phase, stream=None):
        if side_by_side:
            here = torch.cuda.current_stream()   # (under capture: the capturing stream, which `stream` names)
            branch.wait_stream(here)
            capi.marlin_gemm_batch(wide[phase], torch.bfloat16, UINT4, scratch, stream=here.cuda_stream)
            capi.marlin_gemm_batch(narrow[phase], torch.bfloat16, UINT4, scratch_b, stream=branch.cuda_stream)
            here.wait_stream(branch)
            return 2
        if slice_copies is None:
            capi.marlin_gemm_batch(tables[phase], torch.bfloat16, UINT4, scratch, signal=signal, stream=stream)
        else:
            capi.marlin_gemm_batch(tables[phase], torch.bfloat16, UINT4, scratch, stream=stream)
            capi.peer_broadcast(slice_copies[phase % 2], world - 1, signal=signal, stream=stream)
        if group is not None:
            group.wait(stream=stream)
        # two classes of token tile (M <= 16, M = 64), one launch each (+ the slice broadcast) + the flag wait
        return 2 + (0 if group is None else 1 + (1 if slice_copies is not None else 0))

    def step_per_gemm(phase, stream=None):
        for i, g in enumerate(singles[phase]):
            last = i == len(keys) - 1 and slice_copies is None
            capi.marlin_gemm_placed(g, torch.bfloat16, UINT4, scratch, signal=signal if last else None, stream=stream)
        if slice_copies is not None:
            capi.peer_broadcast(slice_copies[phase % 2], world - 1, signal=signal, stream=stream)
        if group is not None:
            group.wait(stream=stream)
        return len(keys) + (0 if group is None else 1 + (1 if slice_copies is not None else 0))

    def capture(step_fn):
        """The step as CUDA graphs, one per weight-copy phase, so that replays keep rotating the weights."""
        for phase in range(phases):   # outside any graph first: function attributes, tensor maps
            step_fn(phase)
        torch.cuda.synchronize()
        d.barrier()
        graphs, launches = [], 0
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for phase in range(phases):
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=side):
                    launches = step_fn(phase, stream=side.cuda_stream)
                graphs.append(g)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        return graphs, launches

    def check_status(what):
        torch.cuda.synchronize()
        assert capi.scratch_status(scratch) == 0, f"{what}: a GEMM kernel gave up on a wait: " \
                                                  f"{scratch[:192].view(torch.int32).tolist()}"
        if side_by_side:
            assert capi.scratch_status(scratch_b) == 0, f"{what}: a GEMM kernel gave up on a wait: " \
                                                        f"{scratch_b[:192].view(torch.int32).tolist()}"
        if group is not None:
            assert group.wait_status() == (0, 0), f"{what}: a wait for a peer's completion flag ran out: {group.wait_status()}"

    counter = [0]

    def replayer(graphs):
        def run(n):
            for _ in range(n):
                graphs[counter[0] % phases].replay()
                counter[0] += 1
        return run

    warmup = max(args.warmup, 3)
    repeats = 5
    graphs, launches_per_step = capture(step_batched)
    run = replayer(graphs)
    run(max(warmup, phases))   # every graph at least once before anything is timed
    check_status("warm-up")
    with ClockSampler(d.local_rank) as clocks:
        time.sleep(0.15)
        regions = timed_regions(d, run, args.steps, repeats)
        time.sleep(0.15)
    check_status("timed region")
    ms_per_step = statistics.median(regions)
    last_phase = (counter[0] - 1) % phases

    # ---- N > 1: what arrived from every rank must be what that rank's shard computes ---------------
    checked = None
    if group is not None:
        checked = check_gathered(d, capi, layers, acts, keys, outs[last_phase % 2], last_phase, scratch, full_n, full_k)

    # ---- the same step as sixteen separate launches -------------------------------------------------
    per_gemm = None
    if not args.headline_only:
        graphs16, launches16 = capture(step_per_gemm)
        run16 = replayer(graphs16)
        run16(max(warmup, phases))
        reg16 = timed_regions(d, run16, args.steps, 3)
        check_status("per-GEMM step")
        per_gemm = {"ms_per_step": statistics.median(reg16), "launches_per_step": launches16,
                    "note": "the same 16 GEMMs as one launch each (programmatic dependent launches in a graph)"}
        del graphs16

    # ---- end to end through the operator call with host buffers -------------------------------
    multi = None if group is None else {"group": group, "offsets": offsets, "outs": outs, "signal": signal,
                                        "scratch": scratch, "set_bytes": set_bytes}
    e2e = e2e_decode(d, args, layers, acts, keys, full_n, phases, multi)
    check_status("end-to-end step")

    step_weight_bytes = sum(weight_bytes(k, n) for _, k, n in SHAPES) * len(MS)
    step_algo_bytes = sum(algorithmic_bytes(m, k, n // world) for _, k, n in SHAPES for m in MS)  # per GPU
    value = step_weight_bytes / (ms_per_step * 1e-3) / 1e9
    achieved = step_algo_bytes / (ms_per_step * 1e-3) / 1e9
    if per_gemm is not None:
        per_gemm["value"] = step_weight_bytes / (per_gemm["ms_per_step"] * 1e-3) / 1e9
        per_gemm["roofline_frac"] = step_algo_bytes / (per_gemm["ms_per_step"] * 1e-3) / 1e9 / peaks["hbm"]

    result = {
        "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world,
        "steps": args.steps, "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD,
                   "parallelism": "single GPU" if world == 1 else
                   f"column-parallel N-shard x{world}; " +
                   ("the GEMM epilogue stores each slice into every rank's full-width result over NVLink"
                    if slice_copies is None else
                    "one copy launch behind the GEMMs stores every slice into the other ranks' full-width results over NVLink") +
                   " (peer-mapped buffers), completion flags + bounded wait per step",
                   "l2": f"inputs larger than L2: {copies} full weight copies "
                         f"({copies * layer_bytes / 1e6:.0f} MB per GPU) used in rotation",
                   "launch": "CUDA graph replay of the step; the 16 problems as two batched persistent launches" +
                             (", side by side on two streams" if side_by_side else "")},
        "timing": dict(spread_of(regions), unit="ms per step", note=f"{repeats} timed regions of {args.steps} steps, "
                       "CUDA events, max over ranks per region; `ms_per_step` is the median"),
        "e2e": e2e,
        "gpu_launches": launches_per_step * args.steps * repeats,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm"], "unit": "GB/s",
                     "frac": achieved / peaks["hbm"], "peak_kind": f"of {peaks['kind']}",
                     "traffic": TRAFFIC_BYTES_PER_STEP if world == 1 else None,
                     "traffic_unit": "DRAM bytes per step, scaled from one ncu capture of the kernel",
                     "kernel": "W4A16GemmBatchKernel", "algorithmic_bytes_per_step": step_algo_bytes},
        "clocks": clocks.summary(),
    }
    if checked is not None:
        result["checked"] = checked
    if per_gemm is not None:
        result["per_gemm"] = per_gemm
    if not args.headline_only:
        del graphs
        layers_keep = layers[0]
        layers = None
        torch.cuda.empty_cache()
        result["prefill"] = bench_prefill(d, group)
        result["moe"] = bench_moe(d, args)
        if world == 1:
            result["small_kernels"] = bench_small(d)
        layers = [layers_keep]
    if rank == 0:
        if world == 1 and not args.no_cpu_baseline:
            result["cpu_baseline"] = cpu_baseline(layers[0], sample_ms=MS, repeats=12)
        print(json.dumps(result), flush=True)
    if world > 1:
        _shutdown(d, group)


# DRAM bytes (read + write) of the GEMM launches of one step.  From the ncu capture of the batched
# launch of the step's twelve M <= 16 problems (profiles/w4a16_gemm_batch_decode_step.md): 349.25 MB
# measured against 342.86 MB algorithmic, ratio 1.019; the M = 64 launch streams its weights once in
# the same way, so the step's traffic is taken as its algorithmic bytes times that ratio (single GPU).
TRAFFIC_BYTES_PER_STEP = int(465084416 * 349.25 / 342.86)


def check_gathered(d, capi, layers, acts, keys, gathered, phase, scratch, full_n, full_k):
    """Every rank recomputes, for every rank r, the step's 16 problems on r's shard (regenerated
    from its seed) as the same batched call, and compares the result with the slice that r stored
    into this rank's full-width matrices: equal bit for bit, or the exchange or the kernel is wrong."""
    ok = True
    for r in range(d.world):
        shard = [make_layer(r, d.world, d.device, phase * len(MS) + mi) for mi in range(len(MS))]
        local = {key: torch.full((key[1], full_n[key[0]] // d.world), float("nan"), dtype=torch.bfloat16, device=d.device)
                 for key in keys}
        problems = []
        for name, m in keys:
            w = shard[MS.index(m)][name]
            problems.append(capi.gemm_problem(acts[(name, m)], w["marlin"], None, w["scales"], w["zeros"],
                                              local[(name, m)], m, w["n"], w["k"]))
        capi.marlin_gemm_batch(capi.problem_array(problems), torch.bfloat16, UINT4, scratch)
        torch.cuda.synchronize()
        for key in keys:
            width = full_n[key[0]] // d.world
            ok = ok and torch.equal(gathered[key][:, r * width:(r + 1) * width], local[key])
        del shard
    return d.all_true(ok)


def e2e_decode(d, args, layers, acts, keys, full_n, phases, multi=None):
    """The step with pinned host activations copied in and the full-width result copied out to pinned host
    memory, inside the timed region.  One GPU: through the public operator (`infini.ops.marlin_gemm`), one
    call per GEMM.  N > 1 (the reference's operator has no placement arguments and the reference no
    communication layer): one C-ABI call per GEMM (`infiniops_b200_marlin_gemm_placed`), whose epilogue
    stores the rank's slice into every rank's full-width result; then the bounded flag wait and the copy out."""
    import infini.ops
    from infiniops_b200 import capi

    if multi is not None:
        return e2e_decode_placed(d, args, layers, acts, keys, full_n, phases, multi)
    assert d.world == 1
    device = d.device
    # One pinned arena for the step's activations and one for its results (and the same on the device),
    # so that a step moves its inputs in one host -> device copy and its results in one device -> host copy
    # instead of sixteen small ones each; the operator calls take views of the arenas.
    def arena(shapes, **kw):
        sizes = [-(-(r * c) // 128) * 128 for r, c in shapes.values()]   # 256-byte aligned slices
        flat = torch.empty(sum(sizes), dtype=torch.bfloat16, **kw)
        views, at = {}, 0
        for (key, (r, c)), size in zip(shapes.items(), sizes):
            views[key] = flat[at:at + r * c].view(r, c)
            at += size
        return flat, views

    in_shapes = {key: tuple(acts[key].shape) for key in keys}
    out_shapes = {key: (key[1], full_n[key[0]]) for key in keys}

    class Lane:
        """One set of step buffers (pinned host arenas and their device twins) with a stream of its own."""

        def __init__(self):
            self.host_in_flat, self.host_in = arena(in_shapes, pin_memory=True)
            self.host_out_flat, self.host_out = arena(out_shapes, pin_memory=True)
            self.dev_in_flat, self.dev_in = arena(in_shapes, device=device)
            self.dev_out_flat, self.dev_out = arena(out_shapes, device=device)
            for key in keys:
                self.host_in[key].copy_(acts[key])
            self.workspace = torch.zeros(432, dtype=torch.int32, device=device)
            self.stream = torch.cuda.Stream()
            self.graphs = None
            self.last_phase = 0

    # Several lanes (three by default), so that a step's copies overlap the GEMMs of the steps before /
    # after it on the other lanes, and the blocks of one lane's next GEMM fill the SMs that the tail of
    # another lane's GEMM leaves idle (what a host with a few requests in flight does); every step still
    # moves its own inputs in and its own results out inside the timed region.
    lanes = [Lane() for _ in range(max(1, args.e2e_lanes))]
    h2d = lanes[0].host_in_flat.numel() * 2
    d2h = lanes[0].host_out_flat.numel() * 2

    def step(lane, phase):
        stream = torch.cuda.current_stream().cuda_stream
        lane.dev_in_flat.copy_(lane.host_in_flat, non_blocking=True)
        for name, m in keys:
            w = layers[phase * len(MS) + MS.index(m)][name]
            infini.ops.marlin_gemm(lane.dev_in[(name, m)], w["marlin"], None, w["scales"], None, None, w["zeros"], None,
                                   None, lane.workspace, UINT4, m, w["n"], w["k"], True, False, True, False,
                                   lane.dev_out[(name, m)], stream=stream)
        lane.host_out_flat.copy_(lane.dev_out_flat, non_blocking=True)

    for i in range(max(3, phases)):
        step(lanes[0], i % phases)
    torch.cuda.synchronize()
    steps = max(3, min(args.steps, 50))
    count = [0]
    # One CUDA graph per lane and weight-copy phase holding the step as the caller issues it: a
    # host -> device copy node, the operator's sixteen launches, a device -> host copy node.  Each
    # lane is captured on its own stream: the operator keeps its split-K scratch per stream, so the
    # lanes' GEMMs never share one.
    for lane in lanes:
        lane.stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(lane.stream):
            step(lane, 0)   # outside capture first: the operator's per-stream scratch is allocated on first use
            torch.cuda.synchronize()
            lane.graphs = []
            for phase in range(phases):
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=lane.stream):
                    step(lane, phase)
                lane.graphs.append(g)
        torch.cuda.current_stream().wait_stream(lane.stream)
    torch.cuda.synchronize()

    def run(n):
        # the timing events sit on the current stream: the lanes start after it and it ends after them
        main = torch.cuda.current_stream()
        for lane in lanes:
            lane.stream.wait_stream(main)
        for _ in range(n):
            lane = lanes[count[0] % len(lanes)]
            with torch.cuda.stream(lane.stream):
                lane.graphs[count[0] % phases].replay()
            lane.last_phase = count[0] % phases
            count[0] += 1
        for lane in lanes:
            main.wait_stream(lane.stream)

    run(2 * len(lanes))
    torch.cuda.synchronize()
    regions = timed_regions(d, run, steps, 3)
    ms = statistics.median(regions)
    torch.cuda.synchronize()
    for lane in lanes:
        # what came back to the host must be what the device computed ...
        assert torch.equal(lane.host_out[keys[-1]], lane.dev_out[keys[-1]].cpu()), "e2e: host result differs"
        # ... and what a lone call of the same GEMM computes (the lanes' launches ran side by side)
        for name, m in (keys[0], keys[-1]):
            w = layers[lane.last_phase * len(MS) + MS.index(m)][name]
            alone = torch.empty_like(lane.dev_out[(name, m)])
            capi.marlin_gemm(acts[(name, m)], w["marlin"], None, w["scales"], w["zeros"], UINT4, m, w["n"], w["k"], alone)
            assert torch.equal(alone, lane.dev_out[(name, m)]), "e2e: result differs from the GEMM run alone"
    step_weight_bytes = sum(weight_bytes(k, n) for _, k, n in SHAPES) * len(MS)
    return {"value": step_weight_bytes / (ms * 1e-3) / 1e9, "unit": "GB/s", "h2d_bytes_per_step": h2d,
            "d2h_bytes_per_step": d2h, "steps": steps, "ms_per_step": ms,
            "note": "infini.ops.marlin_gemm per GEMM; the step's activations in one copy from pinned host memory, its results "
                    f"in one copy back to pinned host memory; the step (copies and operator calls) replayed as a CUDA graph, "
                    f"steps alternating between {len(lanes)} sets of buffers and streams so that one step's copies and "
                    "launch tails overlap the others' GEMMs"}


def e2e_decode_placed(d, args, layers, acts, keys, full_n, phases, multi):
    """`e2e` at N > 1: host activations in (one pinned copy), sixteen placed GEMM calls whose epilogues
    store into every rank's result set, the flag wait, the full-width results out (one pinned copy).

    Three streams per rank -- copy in, GEMMs, copy out -- with two input buffers and the two result sets
    of the device-resident step, which alternate with the step.  What orders them (step i, set s = i % 2):
      * copy in (i) overwrites input buffer s, last read by the GEMMs of step i - 2;
      * set s is written by every rank's GEMMs (i), copied out by (i), and written again by the GEMMs
        (i + 2) -- the peers' as soon as this rank has signalled step i + 1.  So the copy out (i) must be
        over before this rank's last GEMM of step i + 1, the one that raises the signal: the step is two
        CUDA graphs per weight-copy phase, fifteen GEMMs / the last GEMM + flag wait, with the wait for
        the copy out (i - 1) between them."""
    from infiniops_b200 import capi

    world, rank, device = d.world, d.rank, d.device
    group, offsets, outs, signal, scratch = (multi[k] for k in ("group", "offsets", "outs", "signal", "scratch"))
    sizes = [-(-(m * acts[(name, m)].shape[1]) // 128) * 128 for name, m in keys]
    host_in = torch.empty(sum(sizes), dtype=torch.bfloat16, pin_memory=True)
    dev_in = [torch.empty(sum(sizes), dtype=torch.bfloat16, device=device) for _ in range(2)]
    views, at = [{}, {}], 0
    for key, size in zip(keys, sizes):
        r, c = acts[key].shape
        for s in range(2):
            views[s][key] = dev_in[s][at:at + r * c].view(r, c)
        host_in[at:at + r * c].view(r, c).copy_(acts[key])
        at += size
    # a result set is one contiguous piece of the arena (carved key by key, 256-byte aligned)
    sets = [group.local(offsets[s][keys[0]], (multi["set_bytes"],), torch.uint8) for s in range(2)]
    host_out = [torch.empty(multi["set_bytes"], dtype=torch.uint8, pin_memory=True) for _ in range(2)]
    assert phases % 2 == 0   # so that a phase always meets the same buffers: phase % 2 == step % 2

    def problem(phase, key):
        name, m = key
        w = layers[phase * len(MS) + MS.index(m)][name]
        peers = [group.address(r, offsets[phase % 2][key]) for r in group.others()]
        return capi.gemm_problem(views[phase % 2][key], w["marlin"], None, w["scales"], w["zeros"], outs[phase % 2][key],
                                 m, w["n"], w["k"], out_ld=full_n[name], out_col0=rank * w["n"], peer_out=peers)

    problems = [[problem(phase, key) for key in keys] for phase in range(phases)]

    def gemms(phase, part, stream=None):
        """part 0: all GEMMs but the last; part 1: the last one (it raises the signal) and the flag wait."""
        todo = problems[phase][:-1] if part == 0 else problems[phase][-1:]
        for g in todo:
            capi.marlin_gemm_placed(g, torch.bfloat16, UINT4, scratch, signal=signal if part == 1 else None, stream=stream)
        if part == 1:
            group.wait(stream=stream)

    for phase in range(phases):   # outside any graph first, one stream, copies in step order
        dev_in[phase % 2].copy_(host_in, non_blocking=True)
        gemms(phase, 0)
        gemms(phase, 1)
        host_out[phase % 2].copy_(sets[phase % 2], non_blocking=True)
    torch.cuda.synchronize()
    d.barrier()
    copy_in, compute, copy_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
    graphs = []
    compute.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(compute):
        for phase in range(phases):
            pair = []
            for part in range(2):
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=compute):
                    gemms(phase, part, stream=compute.cuda_stream)
                pair.append(g)
            graphs.append(pair)
    torch.cuda.current_stream().wait_stream(compute)
    torch.cuda.synchronize()
    # (captured graphs have not run: every rank has signalled and waited `phases` times so far)
    in_done = [torch.cuda.Event() for _ in range(2)]
    gemm_done = [torch.cuda.Event() for _ in range(2)]
    out_done = [torch.cuda.Event() for _ in range(2)]
    for e in in_done + gemm_done + out_done:
        e.record()
    torch.cuda.synchronize()
    count = [0]

    def run(n):
        main = torch.cuda.current_stream()
        for st in (copy_in, compute, copy_out):
            st.wait_stream(main)
        for _ in range(n):
            i = count[0]
            s, phase = i % 2, i % phases
            copy_in.wait_event(gemm_done[s])          # the GEMMs of step i - 2 have read input buffer s
            with torch.cuda.stream(copy_in):
                dev_in[s].copy_(host_in, non_blocking=True)
                in_done[s].record()
            compute.wait_event(in_done[s])
            with torch.cuda.stream(compute):
                graphs[phase][0].replay()
            # set 1 - s (step i - 1) is on the host before this rank's signal lets the peers write it again
            # (and this rank's own GEMMs of step i + 1 follow this point in the stream)
            compute.wait_event(out_done[1 - s])
            with torch.cuda.stream(compute):
                graphs[phase][1].replay()
                gemm_done[s].record()
            copy_out.wait_event(gemm_done[s])
            with torch.cuda.stream(copy_out):
                host_out[s].copy_(sets[s], non_blocking=True)
                out_done[s].record()
            count[0] += 1
        for st in (copy_in, compute, copy_out):
            main.wait_stream(st)

    run(phases)
    torch.cuda.synchronize()
    steps = max(3, min(args.steps, 50))
    regions = timed_regions(d, run, steps, 3)
    ms = statistics.median(regions)
    torch.cuda.synchronize()
    last = (count[0] - 1) % 2
    assert torch.equal(host_out[last], sets[last].cpu()), "e2e: host result differs"
    step_weight_bytes = sum(weight_bytes(k, n) for _, k, n in SHAPES) * len(MS)
    return {"value": step_weight_bytes / (ms * 1e-3) / 1e9, "unit": "GB/s", "h2d_bytes_per_step": host_in.numel() * 2,
            "d2h_bytes_per_step": multi["set_bytes"], "steps": steps, "ms_per_step": ms,
            "note": "per rank: the step's activations in one copy from pinned host memory, one "
                    "infiniops_b200_marlin_gemm_placed call per GEMM (the epilogue stores the slice into every rank's "
                    "full-width result), the bounded flag wait, the full-width results in one copy back to pinned host "
                    "memory; GEMMs replayed as CUDA graphs, the copies on streams of their own beside the neighbouring "
                    "steps' GEMMs"}


# ---------------------------------------------------------------------------------------------------
def bench_prefill(d, group):
    """configs[2]: the four linears at M = 4096, GPTQ-symmetric, bf16.  TFLOP/s per linear and for the four
    together, against the measured bf16 burst peak (the fraction of the sustained figure is reported beside
    it); every linear is timed as short runs of back-to-back launches.  With N > 1 every
    rank computes its column shard and the epilogue stores it into every rank's full-width result."""
    from infiniops_b200 import capi

    world, rank, device = d.world, d.rank, d.device
    peaks = measured_peaks()
    m = 4096
    out = {"metric": "W4A16 GEMM TFLOP/s (prefill, M=4096)", "unit": "TFLOP/s", "linears": {},
           "workload": "configs[2]: qkv, o, gate_up, down at M=4096, GPTQ symmetric int4, g=128, bf16"}
    gen = torch.Generator(device=device).manual_seed(SEED + 2000 + rank)
    total_ms, total_flops = 0.0, 0
    if group is not None:
        off = group.carve(m * 28672 * 2)
    sets = 3   # activations / results in rotation: A + C of a linear are 67..270 MB, three sets exceed the 126 MB L2
    reps = 6
    for name, k, n in SHAPES:
        n_local = n // world
        marlin = torch.randint(-2**31, 2**31 - 1, (k // 16, 2 * n_local), dtype=torch.int32, device=device, generator=gen)
        scales = (torch.randn((k // GROUP, n_local), device=device, generator=gen).abs() * 0.01 + 1e-3).bfloat16()
        acts = [torch.randn((m, k), device=device, generator=gen).bfloat16() for _ in range(sets)]
        if group is None:
            fulls = [torch.empty((m, n), dtype=torch.bfloat16, device=device) for _ in range(sets)]
            peers = [[]] * sets
        else:   # one peer-mapped result matrix (the largest linear alone is 235 MB, more than L2)
            fulls = [group.local(off, (m, n), torch.bfloat16)] * sets
            peers = [[group.address(r, off) for r in group.others()]] * sets
        problems = [capi.gemm_problem(acts[i], marlin, None, scales, None, fulls[i], m, n_local, k, out_ld=n,
                                      out_col0=rank * n_local, peer_out=peers[i]) for i in range(sets)]
        scratch = torch.zeros(capi.lib().infiniops_b200_marlin_gemm_scratch_bytes(m, n_local, k), dtype=torch.uint8,
                              device=device)
        signal = None if group is None else group.signal()

        def launch(i):
            capi.marlin_gemm_placed(problems[i % sets], torch.bfloat16, UINT4B8, scratch, signal=signal)
            if group is not None:
                group.wait()

        for i in range(3):
            launch(i)

        def run(count):
            for i in range(count):
                launch(i)

        times = timed_regions(d, run, reps, 5)   # ms per launch, back to back as in a prefill pass
        torch.cuda.synchronize()
        assert capi.scratch_status(scratch) == 0
        ms = statistics.median(times)
        flops = 2 * m * k * n
        out["linears"][f"{name} {k}x{n}"] = {"ms": ms, "tflops": flops / (ms * 1e-3) / 1e12,
                                             "frac_of_bf16_peak": flops / (ms * 1e-3) / 1e12 / (peaks["bf16"] * world)}
        total_ms += ms
        total_flops += flops
        del marlin, scales, acts, fulls, problems, scratch
    out["value"] = total_flops / (total_ms * 1e-3) / 1e12
    out["ms_per_step"] = total_ms
    out["roofline"] = {"bound": "tensor", "achieved": out["value"] / world, "peak": peaks["bf16"], "unit": "TFLOP/s",
                       "frac": out["value"] / world / peaks["bf16"], "peak_kind": f"of {peaks['kind']} (burst), per GPU",
                       "frac_of_sustained": out["value"] / world / peaks["bf16_sustained"]}
    out["timing"] = ("per linear: 5 regions of 6 back-to-back launches over 3 sets of activations and results in rotation "
                     "(inputs larger than L2), CUDA events, max over ranks; median")
    return out


MOE_CONFIGS = {
    "mixtral": {"experts": 8, "top_k": 2, "hidden": 4096, "inter": 14336, "zeros": False, "router": "softmax",
                "label": "configs[3]: Mixtral-8x7B-shaped MoE layer, E=8 top-2 H=4096 I=14336, GPTQ symmetric"},
    "deepseek": {"experts": 256, "top_k": 8, "hidden": 7168, "inter": 2048, "zeros": True, "router": "grouped",
                 "label": "configs[4]: DeepSeek-V3-shaped MoE layer, E=256 top-8 (8 groups, 4 kept, sigmoid + bias) "
                          "H=7168 I=2048, AWQ zero points"},
}


def moe_problem(cfg, tokens, d):
    """Expert weights of this rank (random Marlin words: the repack is measured on its own), tokens and
    router inputs of this rank."""
    from infiniops_b200 import moe_layer

    dev = d.device
    e_local = cfg["experts"] // d.world
    t_local = max(1, tokens // d.world)
    gen = torch.Generator(device=dev).manual_seed(SEED + 3000 + d.rank)

    def packed(k, n):
        w = torch.empty((e_local, k // 16, 2 * n), dtype=torch.int32, device=dev)
        for e in range(e_local):
            w[e] = torch.randint(-2**31, 2**31 - 1, (k // 16, 2 * n), dtype=torch.int32, device=dev, generator=gen)
        s = (torch.randn((e_local, k // GROUP, n), device=dev, generator=gen).abs() * 0.01 + 1e-3).bfloat16()
        z = torch.randint(-2**31, 2**31 - 1, (e_local, k // GROUP, n // 8), dtype=torch.int32, device=dev,
                          generator=gen) if cfg["zeros"] else None
        return w, s, z

    w13, s13, z13 = packed(cfg["hidden"], 2 * cfg["inter"])
    w2, s2, z2 = packed(cfg["inter"], cfg["hidden"])
    weights = moe_layer.ExpertWeights(w13, s13, z13, w2, s2, z2, cfg["hidden"], cfg["inter"])
    x = torch.randn((t_local, cfg["hidden"]), device=dev, generator=gen).bfloat16()
    logits = torch.randn((t_local, cfg["experts"]), device=dev, generator=gen)
    bias = torch.randn(cfg["experts"], device=dev, generator=gen) * 0.1
    return weights, x, logits, bias, t_local


def moe_layer_time(d, cfg, tokens, steps, warmup, block=64, fuse=None):
    """ms per layer pass (router -> sort -> w13 GEMM -> silu_and_mul -> w2 GEMM -> moe_sum, with dispatch and
    combine when sharded), median of 3 regions."""
    from infiniops_b200 import capi, moe_layer, parallel

    weights, x, logits, bias, t_local = moe_problem(cfg, tokens, d)
    # routing block: 64 as BASELINE.json's chain states it, or chosen from the rows per expert
    fused = False
    block_arg = block
    if block == 0:
        block = moe_layer.routing_block(t_local * d.world * cfg["top_k"] // d.world, weights.num_experts,
                                        cfg["hidden"] * cfg["inter"])
        # (silu_and_mul inside the first GEMM's epilogue -- `--moe-fuse silu` -- is not part of this arm:
        # it measured 2-4 % slower than the separate pass at every size once all GEMM stores are tiles)
    if fuse is not None:
        fused = fuse in ("silu", "all")
    # router + sort as one launch: one thread block routes all tokens, so only for a handful of them
    fuse_router = (block_arg == 0 and t_local <= 32) if fuse is None else fuse in ("router", "all")
    weights.interleaved = fused
    runner = moe_layer.RoutedExperts(weights, block)
    launches = [0]
    ep = None
    if d.world > 1:
        # device-side expert parallelism: dispatch, expert GEMMs and combine over peer-mapped arenas
        ep = parallel.DeviceExpertParallel(weights, cfg["top_k"], t_local, d.device, block)
    out = torch.empty_like(x)

    def route():
        if cfg["router"] == "softmax":
            return moe_layer.route_softmax(logits, cfg["top_k"])
        return moe_layer.route_grouped(logits, bias, 8, 4, cfg["top_k"], 2.5)

    router = ({"kind": "softmax", "top_k": cfg["top_k"]} if cfg["router"] == "softmax" else
              {"kind": "grouped", "top_k": cfg["top_k"], "bias": bias, "groups": 8, "topk_group": 4, "scaling": 2.5})

    def step(stream=None):
        sort = 1 if t_local * cfg["top_k"] <= 1024 else 2
        if ep is None and fuse_router and sort == 1:
            # router + sort as one launch, row gather + w13 GEMM (with silu_and_mul), w2 GEMM, moe_sum
            launches[0] = 1 + 2 + (0 if fused else 1) + 1 + 1
            return moe_layer.layer_from_logits(x, logits, router, runner, stream=stream)
        w, ids = route() if stream is None else route_on(stream)
        if ep is None:
            # router, sort, row gather + w13 GEMM, silu_and_mul (unless fused), w2 GEMM, moe_sum
            launches[0] = 1 + sort + 2 + (0 if fused else 1) + 1 + 1
            return moe_layer.single_gpu_layer(x, w, ids, runner, stream=stream)
        # router, plan, dispatch, wait, unpack, sort, w13 GEMM, silu_and_mul (unless fused), w2 GEMM, wait, moe_sum
        launches[0] = 5 + sort + 1 + (0 if fused else 1) + 1 + 2
        return ep(x, ids, w, out=out, stream=stream)

    def route_on(stream):
        if cfg["router"] == "softmax":
            return moe_layer.route_softmax(logits, cfg["top_k"], stream=stream)
        return moe_layer.route_grouped(logits, bias, 8, 4, cfg["top_k"], 2.5, stream=stream)

    for _ in range(max(warmup, 3)):
        step()
    torch.cuda.synchronize()
    d.barrier()
    # the layer as one CUDA graph (nothing in it is read back by the host)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            step(stream=side.cuda_stream)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph.replay()

    def run(n):
        for _ in range(n):
            graph.replay()

    regions = timed_regions(d, run, steps, 3)
    torch.cuda.synchronize()
    assert capi.scratch_status(capi.scratch(d.device, 0)) == 0
    if ep is not None:
        assert ep.status() == (0, 0, 0), f"a wait for a peer's flag ran out: {ep.status()}"
        del graph
        ep.close()
    return statistics.median(regions), t_local * d.world, launches[0], block


def bench_moe(d, args):
    """configs[3] and configs[4]: tokens/s of the whole layer.  Mixtral shape at T = 1024 and 4096, DeepSeek shape
    at T = 512 and 8192 (the largest T of each configuration fits one GPU)."""
    peaks = measured_peaks()
    out = {"metric": "MoE tokens/s", "unit": "tokens/s", "cases": {}}
    for name, token_counts in (("mixtral", (1024, 4096)), ("deepseek", (512, 8192))):
        cfg = MOE_CONFIGS[name]
        if cfg["experts"] % d.world:
            continue
        for tokens in token_counts:
            steps = 10 if tokens <= 1024 else 5
            flops = tokens * cfg["top_k"] * (2 * cfg["hidden"] * 2 * cfg["inter"] + 2 * cfg["inter"] * cfg["hidden"])
            case = {"workload": cfg["label"]}
            # block 64: the chain exactly as BASELINE.json states it; adaptive: the routing block chosen
            # from the rows per expert (16 ... 256) and, with 128- / 256-row blocks, both GEMMs storing
            # tiles in sorted order with the scatter folded into the final sum (same bits as the chain)
            for label, block in (("block64", 64), ("adaptive_block", 0)):
                ms, t_global, launches, used = moe_layer_time(d, cfg, tokens, steps, 3, block)
                tf = flops / (ms * 1e-3) / 1e12
                # the bound is whichever ideal time is longer: the matrix products on the tensor cores, or one
                # pass over the int4 weights of the experts the routes touch (expected number of distinct
                # experts for uniform routing) plus the layer's activations
                touched = cfg["experts"] * (1.0 - (1.0 - 1.0 / cfg["experts"]) ** (tokens * cfg["top_k"]))
                expert_bytes = 3 * cfg["hidden"] * cfg["inter"] // 2 * (1 + 2.5 * 2 / GROUP)
                hbm_bytes = touched * expert_bytes + tokens * cfg["top_k"] * (cfg["hidden"] * 2 + 3 * cfg["inter"]) * 2 * 2
                t_tensor = flops / (peaks["bf16"] * 1e12 * d.world)
                t_hbm = hbm_bytes / (peaks["hbm"] * 1e9 * d.world)
                if t_hbm > t_tensor:
                    gbs = hbm_bytes / (ms * 1e-3) / 1e9
                    roof = {"bound": "hbm", "achieved": gbs / d.world, "peak": peaks["hbm"], "unit": "GB/s",
                            "frac": gbs / d.world / peaks["hbm"], "peak_kind": f"of {peaks['kind']}, per GPU",
                            "note": "weights of the experts touched, read once, + activations"}
                else:
                    roof = {"bound": "tensor", "achieved": tf / d.world, "peak": peaks["bf16"], "unit": "TFLOP/s",
                            "frac": tf / d.world / peaks["bf16"], "peak_kind": f"of {peaks['kind']} (burst), per GPU"}
                case[label] = {"moe_block_size": used, "tokens_per_s": t_global / (ms * 1e-3), "ms_per_layer": ms,
                               "tflops": tf, "launches_per_layer": launches, "roofline": roof}
                torch.cuda.empty_cache()
            best = max(("block64", "adaptive_block"), key=lambda k: case[k]["tokens_per_s"])
            case["tokens_per_s"], case["best"] = case[best]["tokens_per_s"], best
            out["cases"][f"{name} T={tokens}"] = case
    head = out["cases"].get("mixtral T=4096")
    if head:
        out["value"] = head["tokens_per_s"]
    out["parallelism"] = "single GPU" if d.world == 1 else (f"expert-parallel x{d.world}: token rows stored into the expert owners' "
                                                                "arenas over NVLink, results stored back by the w2 GEMM epilogue, flags + bounded waits")
    return out


def bench_small(d):
    """GB/s of the memory-bound kernels at their layer sizes, against the measured HBM bandwidth.  Each launch
    is timed on its own with the L2 flushed before it (median of 7)."""
    from infiniops_b200 import capi

    dev = d.device
    peaks = measured_peaks()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    gen = torch.Generator(device=dev).manual_seed(SEED + 5000)
    out = {}

    def measure(name, nbytes, launch, note):
        for _ in range(2):
            launch()
        times = []
        for _ in range(7):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            launch()
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
        ms = statistics.median(times)
        gbs = nbytes / (ms * 1e-3) / 1e9
        out[name] = {"us": ms * 1e3, "algorithmic_bytes": nbytes, "gbs": gbs, "frac_of_hbm": gbs / peaks["hbm"],
                     "note": note}

    k, n = 4096, 28672
    src = torch.randint(-2**31, 2**31 - 1, (k // 8, n), dtype=torch.int32, device=dev, generator=gen)
    dst = torch.empty((k // 16, 2 * n), dtype=torch.int32, device=dev)
    measure("gptq_marlin_repack", k * n, lambda: capi.gptq_marlin_repack(src, None, k, n, 4, False, dst),
            "4096 x 28672, 4-bit: K*N/2 read + K*N/2 written")
    src2 = torch.randint(-2**31, 2**31 - 1, (k, n // 8), dtype=torch.int32, device=dev, generator=gen)
    measure("awq_marlin_repack", k * n, lambda: capi.awq_marlin_repack(src2, k, n, 4, False, dst), "4096 x 28672, 4-bit")
    del src, src2, dst

    t, e, topk = 4096, 8, 2
    logits = torch.randn((t, e), device=dev, generator=gen)
    w = torch.empty((t, topk), device=dev)
    ids = torch.empty((t, topk), dtype=torch.int32, device=dev)
    tei = torch.empty((t, topk), dtype=torch.int32, device=dev)
    measure("topk_softmax", t * e * 4 + t * topk * 12, lambda: capi.topk_softmax(logits, None, None, True, w, ids, tei),
            "T=4096, E=8, top-2 (launch-latency bound at this size)")
    t, e, topk = 8192, 256, 8
    scores = torch.randn((t, e), device=dev, generator=gen)
    bias = torch.randn(e, device=dev, generator=gen) * 0.1
    w8 = torch.empty((t, topk), device=dev)
    ids8 = torch.empty((t, topk), dtype=torch.int32, device=dev)
    measure("grouped_topk", t * e * 4 + t * topk * 8,
            lambda: capi.grouped_topk(scores, bias, 8, 4, topk, True, 2.5, 1, w8, ids8), "T=8192, E=256, top-8 of 4 of 8 groups")
    capi.grouped_topk(scores, bias, 8, 4, topk, True, 2.5, 1, w8, ids8)
    size = t * topk + e * 63
    sorted_ids = torch.empty(size, dtype=torch.int32, device=dev)
    expert_ids = torch.empty((size + 63) // 64, dtype=torch.int32, device=dev)
    npost = torch.empty(1, dtype=torch.int32, device=dev)
    measure("moe_align_block_size", 4 * (t * topk + size + (size + 63) // 64 + 1),
            lambda: capi.moe_align_block_size(ids8, None, e, 64, sorted_ids, expert_ids, npost),
            "65 536 ids, E=256, block 64 (two launches)")

    rows, inter = 8192, 14336
    x = torch.randn((rows, 2 * inter), device=dev, generator=gen).bfloat16()
    y = torch.empty((rows, inter), dtype=torch.bfloat16, device=dev)
    measure("silu_and_mul", 3 * rows * inter * 2, lambda: capi.silu_and_mul(x, y), "[8192, 2*14336] bf16 (Mixtral, T=4096)")
    del x, y
    t, topk, h = 8192, 8, 7168
    x = torch.randn((t, topk, h), device=dev, generator=gen).bfloat16()
    y = torch.empty((t, h), dtype=torch.bfloat16, device=dev)
    measure("moe_sum", (topk + 1) * t * h * 2, lambda: capi.moe_sum(x, y), "[8192, 8, 7168] bf16 (DeepSeek, T=8192)")
    return out


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
    then-matmul formulation), all host threads, same workload, metric and step definition as the
    repository's arm: one step = the 16 GEMMs (four linears at M in {1, 4, 16, 64})."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    torch.set_num_threads(os.cpu_count() or 1)
    gen_layer = {}
    for si, (name, k, n) in enumerate(SHAPES):
        gen = torch.Generator().manual_seed(SEED + si)
        awq = torch.randint(-2**31, 2**31 - 1, (k, n // 8), dtype=torch.int32, generator=gen)
        scales = (torch.randn((k // GROUP, n), generator=gen).abs() * 0.01 + 1e-3).bfloat16()
        zeros = torch.randint(-2**31, 2**31 - 1, (k // GROUP, n // 8), dtype=torch.int32, generator=gen)
        gen_layer[name] = {"awq": awq, "scales": scales, "zeros": zeros, "n": n}
    problem = cpu_reference_problem(gen_layer)
    warmup = max(args.warmup, 3)
    for _ in range(warmup):
        cpu_pass(problem, MS)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_pass(problem, MS)
    elapsed = time.perf_counter() - t0
    nbytes = sum(weight_bytes(k, n) for _, k, n in SHAPES) * len(MS)
    value = nbytes * args.steps / elapsed / 1e9
    cores = torch.get_num_threads()
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": warmup, "ms_per_step": elapsed / args.steps * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "parallelism": "host cores (rank 0 only)",
                   "launch": "fp32 dequantise + torch matmul per GEMM on the host"},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": cores, "kind": "port",
                         "sample": "every step = the full 16-GEMM step, fp32 dequantise + torch matmul on the host"},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


def run_moe(args):
    """One MoE configuration on its own: `--workload moe --moe-shape mixtral|deepseek --tokens T`."""
    d = Dist(args)
    cfg = MOE_CONFIGS[args.moe_shape]
    with ClockSampler(d.local_rank) as clocks:
        ms, tokens, launches, block = moe_layer_time(d, cfg, args.tokens, min(args.steps, 50), args.warmup, args.moe_block, args.moe_fuse)
    flops = tokens * cfg["top_k"] * (2 * cfg["hidden"] * 2 * cfg["inter"] + 2 * cfg["inter"] * cfg["hidden"])
    if d.rank == 0:
        print(json.dumps({
            "metric": "MoE tokens/s", "value": tokens / (ms * 1e-3), "unit": "tokens/s", "n_gpus": d.world,
            "steps": min(args.steps, 50), "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"{cfg['label']}, T={tokens}", "moe_block_size": block,
                       "parallelism": "single GPU" if d.world == 1 else f"expert-parallel x{d.world}",
                       "l2": "inputs larger than L2: the layer's expert weights"},
            "tflops": flops / (ms * 1e-3) / 1e12, "gpu_launches": launches * min(args.steps, 50) * 3,
            "clocks": clocks.summary()}), flush=True)
    if d.world > 1:
        _shutdown(d, None)


def _shutdown(d, group):
    """Orderly teardown; a watchdog ends the process if the teardown itself blocks -- the result line
    is already out."""
    import gc
    import threading

    import torch.distributed as dist

    threading.Thread(target=lambda: (time.sleep(30), os._exit(0)), daemon=True).start()
    gc.collect()
    torch.cuda.synchronize()
    if group is not None:
        group.close()
    dist.barrier()
    dist.destroy_process_group()


def _moe_sum(capi, routed):
    out = torch.empty((routed.shape[0], routed.shape[2]), dtype=routed.dtype, device=routed.device)
    capi.moe_sum(routed, out)
    return out


def run_one(args):
    """One dense bf16 GEMM `M,K,N` (AWQ with zero points, or GPTQ-symmetric with --gptq), launched a few times
    with an L2 flush in between: the small, self-terminating case used for profiler captures
    (`ncu ... python bench.py --one 16,4096,28672`)."""
    from infiniops_b200 import capi

    m, k, n = (int(v) for v in args.one.split(","))
    dev = torch.device("cuda", 0)
    gen = torch.Generator(device=dev).manual_seed(SEED)
    marlin = torch.randint(-2**31, 2**31 - 1, (k // 16, 2 * n), dtype=torch.int32, device=dev, generator=gen)
    scales = (torch.randn((k // GROUP, n), device=dev, generator=gen).abs() * 0.01 + 1e-3).bfloat16()
    zeros = None if args.gptq else torch.randint(-2**31, 2**31 - 1, (k // GROUP, n // 8), dtype=torch.int32, device=dev,
                                                 generator=gen)
    a = torch.randn((m, k), device=dev, generator=gen).bfloat16()
    out = torch.empty((m, n), dtype=torch.bfloat16, device=dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    times = []
    for _ in range(3):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        capi.marlin_gemm(a, marlin, None, scales, zeros, UINT4B8 if args.gptq else UINT4, m, n, k, out)
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1) * 1e3)
    print(json.dumps({"case": args.one, "weights": "gptq symmetric" if args.gptq else "awq with zero points",
                      "us_per_launch_with_launch_gap": times,
                      "algorithmic_bytes": algorithmic_bytes(m, k, n, not args.gptq), "flops": 2 * m * k * n}))


def run_one_batch(args):
    """The batched decode step on its own, a few times (profiling case for the batched kernel):
    `--one-batch S` runs the 16-problem step on linears scaled down by S (1 = full size)."""
    from infiniops_b200 import capi

    shrink = int(args.one_batch)
    dev = torch.device("cuda", 0)
    gen = torch.Generator(device=dev).manual_seed(SEED)
    problems, keep = [], []
    for name, k, n in SHAPES:
        n = max(128, n // shrink // 128 * 128)
        for m in (tuple(int(v) for v in args.ms.split(",")) if args.ms else MS):   # weights of their own for every problem, as in the step (nothing is shared through L2)
            marlin = torch.randint(-2**31, 2**31 - 1, (k // 16, 2 * n), dtype=torch.int32, device=dev, generator=gen)
            scales = (torch.randn((k // GROUP, n), device=dev, generator=gen).abs() * 0.01 + 1e-3).bfloat16()
            zeros = torch.randint(-2**31, 2**31 - 1, (k // GROUP, n // 8), dtype=torch.int32, device=dev, generator=gen)
            a = torch.randn((m, k), device=dev, generator=gen).bfloat16()
            out = torch.empty((m, n), dtype=torch.bfloat16, device=dev)
            keep.append((marlin, scales, zeros, a, out))
            problems.append(capi.gemm_problem(a, marlin, None, scales, zeros, out, m, n, k))
    table = capi.problem_array(problems)
    scratch = torch.zeros(capi.lib().infiniops_b200_marlin_gemm_batch_scratch_bytes(), dtype=torch.uint8, device=dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    times = []
    for _ in range(3):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        capi.marlin_gemm_batch(table, torch.bfloat16, UINT4, scratch)
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1) * 1e3)
    assert capi.scratch_status(scratch) == 0
    print(json.dumps({"case": f"batched step, linears / {shrink}", "us_per_step_with_launch_gap": times}))


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--workload", default="decode", choices=("decode", "moe"),
                        help="decode = the headline W4A16 decode step with its sub-records; moe = one MoE layer case")
    parser.add_argument("--tokens", type=int, default=1024, help="global tokens of the MoE workload")
    parser.add_argument("--moe-shape", default="mixtral", choices=tuple(MOE_CONFIGS))
    parser.add_argument("--moe-block", type=int, default=64, help="routing block of the MoE workload (0 = adaptive)")
    parser.add_argument("--moe-fuse", default=None, choices=("none", "silu", "router", "all"),
                        help="MoE workload: which fused launches to use (default: all with --moe-block 0, else none)")
    parser.add_argument("--one", default=None, help="M,K,N: run this single GEMM three times (profiling case)")
    parser.add_argument("--one-batch", default=None, help="S: the batched step on linears shrunk by S, three times")
    parser.add_argument("--ms", default=None, help="--one-batch: the row counts to include, e.g. 1,4,16")
    parser.add_argument("--gptq", action="store_true", help="--one: GPTQ-symmetric weights instead of AWQ")
    parser.add_argument("--gather", default="auto", choices=("auto", "epilogue", "broadcast"),
                        help="N > 1: slices stored to the peers by the GEMM epilogue, or by one copy launch behind the GEMMs "
                             "(auto: the epilogue)")
    parser.add_argument("--decode-streams", type=int, default=2, choices=(1, 2),
                        help="N = 1: 2 = the step's two batch calls (M = 64 / M <= 16) side by side on two streams, "
                             "1 = one call, its launches one after the other")
    parser.add_argument("--e2e-lanes", type=int, default=3,
                        help="N = 1: sets of step buffers (each with its stream) the end-to-end leg alternates between")
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=100)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", default="ours", choices=("ours", "reference"))
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--headline-only", action="store_true", help="skip the per-GEMM, prefill, MoE and small-kernel "
                                                                      "sub-records")
    args = parser.parse_args()
    if args.one:
        run_one(args)
    elif args.one_batch:
        run_one_batch(args)
    elif args.impl == "reference":
        run_reference(args)
    elif args.workload == "moe":
        run_moe(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
