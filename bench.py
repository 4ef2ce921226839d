"""MoE-layer benchmark: tokens/s of the route-native MXFP4 sparse-expert layer on B200.

    python bench.py --gpus N --steps K --warmup W [--workload NAME] [--tokens T] [--impl reference]

A step is one pass of the whole layer (router projection, routing, schedule, gate/up + SwiGLU,
down, combine) over one batch of seeded synthetic tokens.  `value` is timed with the inputs
resident in HBM: exactly K steps back to back between two CUDA events on the launching stream with
a synchronise on both sides; that block is repeated until half a second of device time has been
measured and the median block is reported, with the spread beside it.  `e2e` is the same metric
through the host-buffer call, host<->device copies inside the timed region.  The `roofline` object
is for the dominant kernel (gate/up) with the whole-layer figure beside it, `parity` checks the
very output the timed configuration produces against the CPU checker, `cpu_baseline` times the CPU
restatement of the reference shaders on this box's host cores, and `extra` holds the other
configurations of the benchmark (decode batch sizes, prefill, the two large layers).
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import statistics
import sys
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from nerve_b200 import synthetic  # noqa: E402
from nerve_b200.clocks import ClockSampler  # noqa: E402

METRIC = "moe_layer_tokens_per_s"
UNIT = "tokens/s"
DTYPE = "fp8_e4m3 x mxfp4_e2m1 -> f32"
MIN_TIMED_SECONDS = 0.5

WORKLOADS = {
    # name -> (config, default tokens, bound)
    "gpt-oss-20b-decode": ("gpt-oss-20b", 64, "hbm"),
    "gpt-oss-20b-prefill": ("gpt-oss-20b-prefill", 4096, "tensor"),
    "gpt-oss-120b": ("gpt-oss-120b", 8192, "tensor"),
    "deepseek-v3": ("deepseek-v3", 16384, "tensor"),
    "tiny": ("tiny", 64, "hbm"),
}


def measured_peaks() -> tuple[dict, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        return json.loads(path.read_text()), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


def kernel_source_hash() -> str:
    """Identifies the expert kernels a DRAM-traffic capture was taken on."""
    h = hashlib.sha256()
    for name in ("experts_tc.cu", "tcgen05.cuh"):
        h.update((ROOT / "nerve_b200" / "csrc" / name).read_bytes())
    return h.hexdigest()[:12]


def captured_traffic(workload: str, tokens: int) -> tuple[dict | None, str]:
    """dram__bytes_read.sum + dram__bytes_write.sum per launch from the ncu captures summarised under
    profiles/ (one table row per kernel). Returns (None, why) when there is no capture of this workload or
    the expert kernels have changed since it was taken."""
    table = ROOT / "profiles" / "dram_traffic_per_launch.md"
    if not table.exists():
        return None, "no capture table"
    found, stale = {}, False
    for line in table.read_text().splitlines():
        cells = [c.strip() for c in line.strip().strip("|").split("|")]
        if len(cells) < 5 or cells[0] != workload or not cells[1].isdigit() or int(cells[1]) != tokens:
            continue
        if cells[4] != kernel_source_hash():
            stale = True
            continue
        found[cells[2]] = int(cells[3].replace(" ", "").replace(",", ""))
    if found:
        return found, "ncu capture of these kernels, profiles/dram_traffic_per_launch.md"
    return None, "the capture under profiles/ predates the current expert kernels" if stale else "no capture of this workload"


def algorithmic_bytes(cfg: synthetic.MoeConfig, tokens: int, distinct: int) -> dict:
    """Bytes a perfect implementation moves per layer call (each selected expert's weights once)."""
    H, I = cfg.hidden, cfg.intermediate
    gate_up = distinct * 2 * H * I * 17 // 32 + tokens * H  # w1 + w3 codes and scales, quantised tokens
    down = distinct * H * I * 17 // 32 + tokens * cfg.total_k * I
    layer = distinct * cfg.expert_weight_bytes + 2 * tokens * H * 2 + cfg.experts * H * 2
    return {"gate_up": gate_up, "down": down, "layer": layer}


def layer_flops(cfg: synthetic.MoeConfig, tokens: int) -> float:
    return 2.0 * tokens * cfg.total_k * 3 * cfg.hidden * cfg.intermediate


# ---- timing ------------------------------------------------------------------------------------------

def timed_blocks(torch, runner, steps, warmup, scratch=None, sample_clocks=False, min_seconds=MIN_TIMED_SECONDS,
                 max_blocks=400):
    """Blocks of exactly `steps` layer calls back to back between two CUDA events on the stream they run
    on, a synchronise on both sides of every block, no per-stage events inside; blocks repeat until
    `min_seconds` of device time. Returns (ms per step of every block, launches per step, clocks)."""
    runner.plan.set_profiling(False)
    stream = torch.cuda.ExternalStream(runner.device.stream(), device=f"cuda:{runner.device.ordinal}")
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(max(warmup, runner.n_banks + 1)):  # every bank's tables are resolved once before timing
        runner.launch_step()
    torch.cuda.synchronize()
    sampler = ClockSampler(runner.device.ordinal) if sample_clocks else None
    if sampler:
        sampler.start()
    blocks, total, launches = [], 0.0, 0
    while (total < min_seconds * 1e3 or not blocks) and len(blocks) < max_blocks:
        if scratch is not None:
            flush_l2(torch, scratch)
        before = runner.plan.launches()
        torch.cuda.synchronize()
        begin.record(stream)
        for _ in range(steps):
            runner.launch_step()
        end.record(stream)
        torch.cuda.synchronize()
        launches = runner.plan.launches() - before
        ms = begin.elapsed_time(end)
        total += ms
        blocks.append(ms / steps)
    clocks = sampler.stop() if sampler else None
    runner.plan.set_profiling(True)
    return blocks, launches, clocks


def profiled_steps(torch, runner, steps, warmup, scratch=None):
    """Per-kernel times: an event pair around every stage and around each expert kernel."""
    runner.plan.set_profiling(True)
    for _ in range(max(warmup, runner.n_banks + 1)):
        runner.step_resident()
    reports = []
    for _ in range(steps):
        if scratch is not None:
            flush_l2(torch, scratch)
        reports.append(runner.step_resident())  # last_report synchronises the stream
    return reports


def flush_l2(torch, scratch):
    scratch.add_(1)  # read + write of a buffer larger than L2
    torch.cuda.synchronize()


def spread(blocks):
    return {"blocks": len(blocks), "ms_median": statistics.median(blocks), "ms_min": min(blocks), "ms_max": max(blocks)}


# ---- parity of the timed configuration -----------------------------------------------------------------

def parity_of(runner, sample_count=24, rank_slice=None):
    """Checks the output of one layer call of `runner` against the CPU checker: routes and logits of the
    whole batch bit for bit, the layer output on a seeded token sample within the stated tolerance."""
    from oracle import sampled

    cfg, case, tokens = runner.cfg, runner.case, runner.tokens
    logits_buf = runner.device.create_resident_buffer(tokens * ((cfg.experts + 1) // 2) * 4)
    runner.plan.layer(tokens, runner.bank, runner.hidden, runner.output, logits=logits_buf, **runner.kw)
    status = runner.plan.status()
    want_logits, want_routes, _ = sampled.routing_for_batch(cfg, case.hidden, case.router_w, case.router_bias, case.select_bias)
    logits_exact = bool(np.array_equal(logits_buf.read(np.uint32).reshape(want_logits.shape), want_logits))
    routes_exact = bool(np.array_equal(runner.read_routes(), want_routes))
    logits_buf.destroy()
    picked = sampled.sample_tokens(tokens, sample_count, seed=tokens)
    want = sampled.layer_on_sample(cfg, case.hidden, want_logits, case.select_bias, picked,
                                   lambda e: synthetic.expert_tensors(cfg, runner.seed, e))
    m = sampled.error_metrics(runner.read_output()[picked], want["output"])
    ok = routes_exact and logits_exact and status == 0 and sampled.within_tolerance(m)
    return {"pass": bool(ok), "routes_exact": routes_exact, "logits_exact": logits_exact, "status_bits": status,
            "rel_l2": m["rel_l2"], "max_abs": m["max_abs"], "max_abs_over_peak": m["max_abs_over_peak"],
            "output_peak": m["peak"], "mismatched_bf16": m["mismatched"], "values": m["count"],
            "sample_tokens": int(len(picked)),
            "tolerance": f"rel_l2 <= {sampled.REL_L2_TOL}, max_abs <= {sampled.MAX_ABS_OVER_PEAK_TOL} of the output peak, "
                         "against the f64-accumulated checker on the same quantised operands"}


# ---- CPU arm --------------------------------------------------------------------------------------------

def cpu_baseline(cfg, tokens, seed, sample_tokens, budget_s=12.0, threads=None):
    """Times the CPU restatement of the reference shaders on a bounded sample of the workload: `sample_tokens`
    tokens first (a probe of the host's speed), then as many tokens of the workload as about `budget_s`
    seconds take, passed over repeatedly if the whole workload takes less."""
    from oracle import moe_oracle as mo

    if threads:
        mo.lib().oracle_set_threads(int(threads))
    probe = _cpu_layer_pass(cfg, tokens, seed, min(tokens, sample_tokens), passes=1)
    rate = probe["value"]
    sample = int(max(1, min(tokens, rate * budget_s)))
    passes = int(max(1, min(50, budget_s * rate / sample)))
    result = _cpu_layer_pass(cfg, tokens, seed, sample, passes)
    # one host core, on a sample a few per cent of that size
    before = mo.lib().oracle_set_threads(1)
    try:
        few = int(max(1, min(tokens, rate * budget_s / (8.0 * max(1, before)))))
        result["single_core_value"] = _cpu_layer_pass(cfg, tokens, seed, few, passes=1)["value"]
    finally:
        mo.lib().oracle_set_threads(before)
    return result


def _cpu_layer_pass(cfg, tokens, seed, sample, passes):
    from oracle import moe_oracle as mo

    case = synthetic.make_case(cfg, sample, seed=seed, with_weights=False)
    rp, ep = mo.router_params_from(cfg), mo.expert_params_from(cfg, tier=0)  # tier 0: the shaders' f32 accumulation order
    logits = mo.linear_bf16(case.hidden, case.router_w, case.router_bias)
    routes, _ = mo.route(rp, logits, case.select_bias)
    used = sorted(set((routes.reshape(-1) & 0xFFFF).tolist()))
    w = synthetic.expert_tensor_lists(cfg, seed, used, placeholder=np.zeros((1, 1), dtype=np.uint8))
    weights = mo.ExpertWeights(*(w[k] for k in synthetic.EXPERT_TENSOR_NAMES))
    t0 = time.perf_counter()
    for _ in range(passes):
        logits = mo.linear_bf16(case.hidden, case.router_w, case.router_bias)
        mo.moe_layer(rp, ep, case.hidden, logits, case.select_bias, weights)
    seconds = time.perf_counter() - t0
    return {"value": passes * sample / seconds, "unit": UNIT, "cores": mo.lib().oracle_max_threads(), "kind": "port",
            "sample": f"{sample} of {tokens} tokens, whole layer, {passes} pass(es), {seconds:.2f} s",
            "sample_tokens": sample}


def run_reference_arm(args, cfg, tokens):
    """The reference has no CPU execution of this layer and its GPU path is Vulkan, so this arm times the CPU
    restatement of its shaders on all the host's cores. Under a multi-process launcher only rank 0 runs; the
    launcher's OMP_NUM_THREADS=1 is overridden, and the workload is the N ranks' tokens."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    world = max(args.gpus, int(os.environ.get("WORLD_SIZE", "1")))
    tokens = tokens * world  # the GPU arm's weak scaling: every rank brings `tokens` tokens
    cores = os.cpu_count() or 1
    sample_tokens = max(1, min(tokens, args.reference_sample))
    values = []
    budget = min(10.0, 120.0 / max(1, args.warmup + args.steps))  # the whole run stays within a few minutes
    for _ in range(args.warmup + args.steps):
        values.append(cpu_baseline(cfg, tokens, args.seed, sample_tokens, budget_s=budget, threads=cores))
    timed = values[args.warmup:] or values
    value = statistics.mean(v["value"] for v in timed)
    base = dict(timed[-1])
    base["value"] = value
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1e3 * base["sample_tokens"] / value, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": DTYPE, "data": "synthetic",
        "config": workload_config(args, cfg, tokens // world, world),
        "note": "CPU restatement of the reference shaders (the reference has no CPU backend); each step is a "
                "bounded token sample of the workload",
        "cpu_baseline": base,
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def workload_config(args, cfg, tokens, world=1):
    """The same object in both arms' lines: what is computed, not how."""
    return {"workload": args.workload, "tokens": tokens, "tokens_per_rank": tokens, "global_tokens": tokens * world,
            "hidden": cfg.hidden, "intermediate": cfg.intermediate, "experts": cfg.experts, "k": cfg.total_k,
            "parallelism": "single device" if world == 1 else f"ep{world}"}


# ---- one workload on one GPU ------------------------------------------------------------------------------

def roofline_of(cfg, tokens, bound, ms, gate_ms, down_ms, distinct, peaks, peak_kind, probe, workload):
    ab = algorithmic_bytes(cfg, tokens, distinct)
    if bound == "hbm":
        traffic, traffic_note = captured_traffic(workload, tokens)
        achieved = ab["gate_up"] / (gate_ms * 1e-3) / 1e9
        hbm = peaks["hbm_gbs"]
        return {"bound": "hbm", "achieved": achieved, "peak": hbm, "unit": "GB/s", "frac": achieved / hbm,
                "traffic": traffic["gate_up"] if traffic and "gate_up" in traffic else None, "traffic_source": traffic_note,
                "kernel": "gate_up", "peak_kind": f"{peak_kind} STREAM-style copy",
                "algorithmic_bytes_per_launch": ab["gate_up"], "kernel_ms": gate_ms,
                "down_kernel": {"achieved": ab["down"] / (down_ms * 1e-3) / 1e9, "kernel_ms": down_ms,
                                "frac": ab["down"] / (down_ms * 1e-3) / 1e9 / hbm,
                                "traffic": traffic["down"] if traffic and "down" in traffic else None,
                                "algorithmic_bytes_per_launch": ab["down"]},
                "layer": {"achieved": ab["layer"] / (ms * 1e-3) / 1e9, "frac": ab["layer"] / (ms * 1e-3) / 1e9 / hbm,
                          "algorithmic_bytes_per_step": ab["layer"]}}
    flops_gate = 2.0 * tokens * cfg.total_k * 2 * cfg.hidden * cfg.intermediate
    achieved = flops_gate / (gate_ms * 1e-3) / 1e12
    # the denominator is the measured rate of the instruction kind that runs (the tensor-pipe probe of this
    # same process); the cuBLAS bf16 figures are given beside it: the FP8-rate kinds run at twice the bf16
    # rate, mxf4 (which this path cannot use: the reference's activations are E4M3) at four times
    peak = probe["tflops"] if probe else peaks["bf16_tflops"] * 2.0
    kind = ("measured tcgen05.mma kind::mxf8f6f4 block-scaled rate, all SMs, operands in shared memory"
            if probe else f"2 x {peak_kind} cuBLAS bf16 burst rate (no probe)")
    def fracs(tf):
        return {"achieved": tf, "frac": tf / peak, "frac_of_2x_bf16_burst": tf / (peaks["bf16_tflops"] * 2.0),
                "frac_of_mxf4_rate": tf / (2.0 * peak)}
    down_tf = flops_gate / 2.0 / (down_ms * 1e-3) / 1e12
    layer_tf = layer_flops(cfg, tokens) / (ms * 1e-3) / 1e12
    return {"bound": "tensor", **fracs(achieved), "peak": peak, "unit": "TFLOP/s", "traffic": None, "kernel": "gate_up",
            "mma_kind": "mxf8f6f4 (E4M3 activations x E2M1 weights, UE8M0 scale per 32)", "peak_kind": kind,
            "kernel_ms": gate_ms, "flops_per_launch": flops_gate,
            "down_kernel": {**fracs(down_tf), "kernel_ms": down_ms},
            "layer": {**fracs(layer_tf), "flops_per_step": layer_flops(cfg, tokens)}}


def measure_workload(torch, args, workload, tokens, peaks, peak_kind, probe, share=None, steps=None, min_seconds=MIN_TIMED_SECONDS,
                     scratch=None, sample_clocks=False, with_e2e=False, parity_tokens=24):
    """Everything the line reports about one configuration on one GPU. Returns (result dict, runner)."""
    from nerve_b200.resident_layer import LayerRunner

    cfg_name, default_tokens, bound = WORKLOADS[workload]
    cfg = synthetic.CONFIGS[cfg_name]
    tokens = tokens or default_tokens
    steps = steps or args.steps
    runner = LayerRunner(cfg, tokens, args.seed, args.expert_path, banks=args.banks, share=share)
    blocks, launches, clocks = timed_blocks(torch, runner, steps, args.warmup, scratch, sample_clocks, min_seconds)
    ms = statistics.median(blocks)
    reports = profiled_steps(torch, runner, min(steps, 10), 3, scratch)
    gate_ms = statistics.mean(rep["gate_up_kernel_ms"] for rep in reports)
    down_ms = statistics.mean(rep["down_kernel_ms"] for rep in reports)
    distinct = reports[-1]["distinct_experts"]
    result = {
        "tokens": tokens, "tokens_per_s": tokens / (ms * 1e-3), "ms_per_step": ms, "timing": spread(blocks),
        "steps_per_block": steps, "launches_per_block": launches, "launches_per_step": launches / steps,
        "distinct_experts": distinct, "expert_path": "tcgen05" if reports[-1]["tensor_path"] else "cuda-cores",
        "roofline": roofline_of(cfg, tokens, bound, ms, gate_ms, down_ms, distinct, peaks, peak_kind, probe, workload),
        "stage_ms": {k: statistics.mean(rep["stage_ms"][k] for rep in reports) for k in reports[-1]["stage_ms"]},
        "profiled_ms_per_step": statistics.mean(rep["total_ms"] for rep in reports),
        "clocks": clocks,
        "l2": (f"inputs larger than L2: {runner.n_banks} resident weight bank(s) visited in turn, "
               f"{runner.cycle_bytes / 1e6:.0f} MB of weights read between two reads of the same bytes"
               + ("; plus a 256 MB buffer rewritten between timed blocks" if scratch is not None else "")),
    }
    if with_e2e:
        runner.plan.set_profiling(False)
        for _ in range(max(3, runner.n_banks + 1)):
            runner.step_host()
        e2e_ms, t_end = [], time.perf_counter() + 0.6 * min_seconds
        while len(e2e_ms) < steps or (time.perf_counter() < t_end and len(e2e_ms) < 5000):
            e2e_ms.append(runner.step_host())
        e2e = statistics.median(e2e_ms)
        result["e2e"] = {"value": tokens / (e2e * 1e-3), "unit": UNIT, "h2d_bytes_per_step": tokens * cfg.hidden * 2,
                         "d2h_bytes_per_step": tokens * cfg.hidden * 2, "ms_per_step": e2e, "calls": len(e2e_ms),
                         "ms_min": min(e2e_ms), "ms_max": max(e2e_ms)}
    if parity_tokens and not args.no_parity:
        result["parity"] = parity_of(runner, parity_tokens)
    return result, runner


def compact(result):
    """The figures of an `extra` entry."""
    r = result["roofline"]
    out = {"tokens": result["tokens"], "tokens_per_s": result["tokens_per_s"], "ms_per_step": result["ms_per_step"],
           "timing": result["timing"], "launches_per_step": result["launches_per_step"],
           "distinct_experts": result["distinct_experts"], "gate_up_kernel_ms": r["kernel_ms"],
           "down_kernel_ms": r["down_kernel"]["kernel_ms"], "stage_ms": result["stage_ms"], "l2": result["l2"]}
    if r["bound"] == "hbm":
        out.update({"bound": "hbm", "layer_hbm_frac": r["layer"]["frac"], "gate_up_hbm_frac": r["frac"],
                    "down_hbm_frac": r["down_kernel"]["frac"]})
    else:
        out.update({"bound": "tensor", "peak_tflops": r["peak"], "peak_kind": r["peak_kind"],
                    "gate_up": {k: r[k] for k in ("achieved", "frac", "frac_of_2x_bf16_burst", "frac_of_mxf4_rate")},
                    "down": {k: r["down_kernel"][k] for k in ("achieved", "frac", "frac_of_2x_bf16_burst", "frac_of_mxf4_rate")},
                    "layer": {k: r["layer"][k] for k in ("achieved", "frac", "frac_of_2x_bf16_burst", "frac_of_mxf4_rate")}})
    if "parity" in result:
        out["parity"] = result["parity"]
    return out


def release(runner, banks_too=True):
    runner.release()
    if banks_too:
        for bank in runner.banks:
            bank.destroy()
        runner.device.close()


def run_single_gpu(args, cfg, tokens, bound):
    import torch

    from nerve_b200.backend import CudaComputeDevice

    torch.cuda.init()
    peaks, peak_kind = measured_peaks()
    # --l2 flush: additionally rewrite a 256 MB buffer between timed blocks (leaves L2 full of dirty lines
    # whose write-back then competes with the first step's reads); default: the rotating weight banks alone
    scratch = torch.empty(256 * 1024 * 1024 // 4, dtype=torch.int32, device="cuda:0") if args.l2 == "flush" else None
    probe = None
    if not args.no_probe:
        dev = CudaComputeDevice(0)
        probe = dev.probe_mma_rate(128, 8192)
        probe["narrow_tile"] = dev.probe_mma_rate(96, 8192)
        dev.close()

    head, runner = measure_workload(torch, args, args.workload, tokens, peaks, peak_kind, probe, scratch=scratch,
                                    sample_clocks=True, with_e2e=True, min_seconds=args.min_seconds)
    line = {
        "metric": METRIC, "value": head["tokens_per_s"], "unit": UNIT, "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": head["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": DTYPE, "data": "synthetic",
        "config": workload_config(args, cfg, tokens),
        "run": {"distinct_experts": head["distinct_experts"], "expert_path": head["expert_path"], "l2": head["l2"],
                "parallelism": "single device"},
        "timing": head["timing"] | {"rule": f"blocks of {args.steps} steps repeated until {args.min_seconds} s of device time; "
                                            "ms_per_step is the median block"},
        "clocks": head["clocks"], "roofline": head["roofline"], "e2e": head["e2e"],
        "gpu_launches": head["launches_per_block"], "launches_per_step": head["launches_per_step"],
        "stage_ms": head["stage_ms"], "profiled_ms_per_step": head["profiled_ms_per_step"],
    }
    if "parity" in head:
        line["parity"] = head["parity"]
    if probe:
        line["tensor_pipe_probe"] = probe

    if not args.no_extra and args.workload == "gpt-oss-20b-decode":
        extra = {}
        small = argparse.Namespace(**{**vars(args), "warmup": 3})
        for t in (1, 8, 32):
            res, r = measure_workload(torch, small, args.workload, t, peaks, peak_kind, probe, share=runner,
                                      steps=max(5, args.steps), min_seconds=0.15, parity_tokens=t)
            extra[f"decode_T{t}"] = compact(res)
            release(r, banks_too=False)
        release(runner)
        runner = None
        for key, workload in (("prefill_T4096", "gpt-oss-20b-prefill"), ("gpt_oss_120b_T8192", "gpt-oss-120b"),
                              ("deepseek_v3_T16384", "deepseek-v3")):
            try:
                big = argparse.Namespace(**{**vars(args), "warmup": 3, "banks": 1 if workload == "deepseek-v3" else args.banks})
                res, r = measure_workload(torch, big, workload, 0, peaks, peak_kind, probe, steps=3, min_seconds=0.1,
                                          parity_tokens=12)
                extra[key] = compact(res)
                release(r)
            except Exception as error:  # the headline line must not depend on an extra
                extra[key] = {"error": f"{type(error).__name__}: {error}"}
        line["extra"] = extra
    if runner is not None:
        release(runner)

    if not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(cfg, tokens, args.seed, args.reference_sample, threads=os.cpu_count())
    print(json.dumps(line))


# ---- N GPUs: the layer expert-sharded over the ranks ------------------------------------------------------------

def ep_timed(torch, dist, layer, step_fn, steps, min_seconds, local):
    """Blocks of exactly `steps` steps back to back between two events on the stream they run on, a barrier and a
    synchronise on both sides of every block, the slowest rank's time; blocks repeat until `min_seconds` of
    device time. Every rank sees the same (all-reduced) times, so every rank stops after the same block."""
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    blocks, total, launches = [], 0.0, 0
    while (total < min_seconds * 1e3 or not blocks) and len(blocks) < 200:
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        before = layer.home.launches() + layer.work.launches()
        start.record(layer.stream)
        for _ in range(steps):
            step_fn()
        stop.record(layer.stream)
        torch.cuda.synchronize()
        dist.barrier()
        t = torch.tensor([start.elapsed_time(stop) / steps], device=f"cuda:{local}")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        launches = layer.home.launches() + layer.work.launches() - before
        blocks.append(float(t.item()))
        total += blocks[-1] * steps
    return blocks, launches


def ep_parity(torch, dist, layer, cfg, tokens, rank, world, local, seed, sample=8):
    """This rank's slice of the global batch against the CPU checker (outside every timed region): routes of all
    its tokens bit for bit, the layer output on a seeded sample of them; the worst rank is reported."""
    from oracle import sampled

    layer.step(dist)
    got = layer.output()
    with torch.cuda.stream(layer.stream):
        layer._route()  # this rank's routes into buffers the host can read (the library's step keeps its own)
    torch.cuda.synchronize()
    case = layer.case
    mine = np.arange(rank * tokens, (rank + 1) * tokens)
    hidden, bias = case.hidden[mine], case.select_bias
    want_logits, want_routes, _ = sampled.routing_for_batch(cfg, hidden, case.router_w, case.router_bias, bias)
    picked = sampled.sample_tokens(tokens, sample, seed=rank)
    want = sampled.layer_on_sample(cfg, hidden, want_logits, bias, picked, lambda e: synthetic.expert_tensors(cfg, seed, e))
    m = sampled.error_metrics(got[picked], want["output"])
    routes_exact = bool(np.array_equal(layer.t_routes.cpu().numpy().view(np.uint32), want_routes))
    overflow = layer.overflowed()
    ok = torch.tensor([1 if (sampled.within_tolerance(m) and routes_exact and not overflow) else 0], device=f"cuda:{local}")
    worst = torch.tensor([m["rel_l2"], m["max_abs_over_peak"], m["max_abs"]], device=f"cuda:{local}", dtype=torch.float64)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    dist.all_reduce(worst, op=dist.ReduceOp.MAX)
    return {"pass": bool(ok.item()), "routes_exact": routes_exact, "rel_l2": float(worst[0]), "max_abs_over_peak": float(worst[1]),
            "max_abs": float(worst[2]), "sample_tokens": int(len(picked)) * world,
            "note": "every rank checks a seeded sample of its own tokens against the CPU checker; worst rank shown"}


def run_expert_parallel(args, cfg, tokens):
    """bench.py --gpus N: the layer expert-sharded over N ranks, tokens per rank fixed (weak scaling); the two
    large layers follow as `extra`, their whole batch split over the ranks (strong scaling)."""
    import torch
    import torch.distributed as dist

    from nerve_b200.expert_parallel import ExpertParallelLayer
    from nerve_b200.resident_layer import L2_BYTES

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    capacity_factor = float(os.environ.get("NVMOE_EP_CAPACITY", "2.0"))
    # enough resident copies of this rank's experts that a step's weights were last read 4 x L2 ago
    per_expert = cfg.expert_weight_bytes
    owned = cfg.experts // world + cfg.always_count
    touched = max(1, min(tokens * world * cfg.total_k, owned)) * per_expert
    banks = args.banks or max(2, min(8, -(-4 * L2_BYTES // touched)))
    # segments bounded at twice the mean rows per peer (NVMOE_EP_CAPACITY=0: the worst case); an overflow is reported
    layer = ExpertParallelLayer(cfg, tokens, rank, world, local, seed=args.seed, expert_path=args.expert_path, banks=banks,
                                dist=dist, mode=os.environ.get("NVMOE_EP_MODE", "auto"), capacity_factor=capacity_factor)
    for _ in range(max(args.warmup, 3, banks + 1)):
        layer.step(dist)
    torch.cuda.synchronize()
    dist.barrier()
    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.start()
    blocks, launches = ep_timed(torch, dist, layer, lambda: layer.step(dist), args.steps, MIN_TIMED_SECONDS, local)
    clocks = sampler.stop() if sampler else None
    # end to end: tokens start in pinned host memory, the result is read back
    host_in = torch.from_numpy(layer.hidden_host.view(np.int16)).pin_memory()
    host_out = torch.empty((tokens, cfg.hidden), dtype=torch.int16).pin_memory()

    def host_step():
        with torch.cuda.stream(layer.stream):
            layer.t_hidden.copy_(host_in, non_blocking=True)
            layer.step(dist)
            host_out.copy_(layer.t_output, non_blocking=True)

    e2e_blocks, _ = ep_timed(torch, dist, layer, host_step, args.steps, 0.2, local)
    ms, e2e_ms = statistics.median(blocks), statistics.median(e2e_blocks)
    overflow = torch.tensor([1 if layer.overflowed() else 0], device=f"cuda:{local}")
    dist.all_reduce(overflow, op=dist.ReduceOp.MAX)
    parity = None if args.no_parity else ep_parity(torch, dist, layer, cfg, tokens, rank, world, local, args.seed)
    headline = {"mode": layer.mode, "segment": layer.segment, "capacity_factor": layer.capacity_factor}
    del layer
    torch.cuda.empty_cache()

    # the layers the expert-parallel configurations are stated for: the whole batch split over the ranks
    extra = {}
    if not args.no_extra and args.workload == "gpt-oss-20b-decode":
        for key, workload in (("ep_gpt_oss_120b", "gpt-oss-120b"), ("ep_deepseek_v3", "deepseek-v3")):
            try:
                big_name, total, _ = WORKLOADS[workload]
                big = synthetic.CONFIGS[big_name]
                if total % world or big.experts % world:
                    raise ValueError(f"{total} tokens or {big.experts} experts do not split over {world} ranks")
                per_rank = total // world
                # building the layer is the step that can fail on one rank alone (memory): the ranks agree on the
                # outcome before any of them enters a collective of the measurement
                big_layer, problem = None, ""
                try:
                    big_layer = ExpertParallelLayer(big, per_rank, rank, world, local, seed=args.seed, expert_path=args.expert_path,
                                                    banks=1, dist=dist, mode=os.environ.get("NVMOE_EP_MODE", "auto"),
                                                    capacity_factor=1.5 if capacity_factor > 0.0 else 0.0)
                except Exception as error:
                    problem = f"{type(error).__name__}: {error}"
                failed = torch.tensor([0 if big_layer is not None else 1], device=f"cuda:{local}")
                dist.all_reduce(failed, op=dist.ReduceOp.MAX)
                if int(failed.item()):
                    del big_layer
                    torch.cuda.empty_cache()
                    extra[key] = {"error": problem or "another rank could not build the layer"}
                    continue
                for _ in range(3):
                    big_layer.step(dist)
                torch.cuda.synchronize()
                big_blocks, big_launches = ep_timed(torch, dist, big_layer, lambda: big_layer.step(dist), 3, 0.1, local)
                big_ms = statistics.median(big_blocks)
                big_overflow = torch.tensor([1 if big_layer.overflowed() else 0], device=f"cuda:{local}")
                dist.all_reduce(big_overflow, op=dist.ReduceOp.MAX)
                entry = {
                    "tokens": total, "tokens_per_rank": per_rank, "experts_per_rank": big.experts // world, "scaling": "strong",
                    "tokens_per_s": total / (big_ms * 1e-3), "ms_per_step": big_ms, "timing": spread(big_blocks),
                    "launches_per_step": big_launches / 3, "exchange": big_layer.mode, "segment_rows": big_layer.segment,
                    "segment_overflow_in_timed_steps": bool(big_overflow.item()),
                    # rows of routed experts that leave a rank, each way: (world - 1) / world of its routed rows on average
                    "all_to_all_bytes_per_direction_per_rank": int(per_rank * big.k * big.hidden * 2 * (world - 1) / world),
                    "layer_tflops": layer_flops(big, total) / (big_ms * 1e-3) / 1e12,
                }
                if not args.no_parity:
                    entry["parity"] = ep_parity(torch, dist, big_layer, big, per_rank, rank, world, local, args.seed, sample=4)
                extra[key] = entry
                del big_layer
                torch.cuda.empty_cache()
            except Exception as error:  # the headline line must not depend on an extra
                extra[key] = {"error": f"{type(error).__name__}: {error}"}
                break  # a rank that failed inside a measurement is no longer in step with the others

    if rank == 0:
        total_tokens = tokens * world
        peaks, kind = measured_peaks()
        achieved = touched / (ms * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": total_tokens / (ms * 1e-3), "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": DTYPE, "data": "synthetic",
            "config": workload_config(args, cfg, tokens, world),
            "run": {
                "experts_per_rank": cfg.experts // world,
                "parallelism": f"ep{world}: experts sharded by contiguous range, tokens data-parallel, "
                               "NCCL all-to-all dispatch and combine",
                "exchange": headline["mode"], "segment_rows": headline["segment"], "capacity_factor": headline["capacity_factor"],
                "segment_overflow_in_timed_steps": bool(overflow.item()),
                "l2": f"inputs larger than L2: {banks} resident weight banks per rank visited in turn, "
                      f"{touched * banks / 1e6:.0f} MB of weights read between two reads of the same bytes"},
            "timing": spread(blocks), "clocks": clocks,
            "e2e": {"value": total_tokens / (e2e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": tokens * cfg.hidden * 2,
                    "d2h_bytes_per_step": tokens * cfg.hidden * 2, "ms_per_step": e2e_ms, "timing": spread(e2e_blocks)},
            "gpu_launches": int(launches), "launches_per_step": launches / args.steps,
            # whole step of one rank against the HBM copy peak: the weights of the experts it owns cross HBM once
            # per step; the exchanges and the small kernels around them are what the fraction leaves out
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": achieved / peaks["hbm_gbs"], "traffic": None, "kernel": "whole step, per rank",
                         "peak_kind": f"{kind} STREAM-style copy", "algorithmic_bytes_per_launch": touched},
        }
        if parity:
            line["parity"] = parity
        if extra:
            line["extra"] = extra
        print(json.dumps(line))
    dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--workload", default="gpt-oss-20b-decode", choices=sorted(WORKLOADS))
    ap.add_argument("--tokens", type=int, default=0)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--expert-path", type=int, default=0, help="0 automatic, 1 CUDA cores, 2 tcgen05")
    ap.add_argument("--reference-sample", type=int, default=16, help="tokens of the CPU arm's first probe")
    ap.add_argument("--no-extra", action="store_true", help="skip the other batch sizes and configurations")
    ap.add_argument("--l2", default="rotate", choices=["rotate", "flush"],
                    help="rotate: inputs larger than L2 (weight banks visited in turn); flush: also rewrite a 256 MB buffer between blocks")
    ap.add_argument("--banks", type=int, default=0, help="resident weight copies visited in turn (0 = enough for 4 x L2 per cycle)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-parity", action="store_true", help="skip the check of the timed output against the CPU checker")
    ap.add_argument("--no-probe", action="store_true", help="skip the tensor-pipe peak probe")
    ap.add_argument("--min-seconds", type=float, default=MIN_TIMED_SECONDS,
                    help="device time the timed blocks of --steps steps are repeated for (0: one block, for a profiler capture)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "native" else args.warmup

    cfg_name, default_tokens, bound = WORKLOADS[args.workload]
    cfg = synthetic.CONFIGS[cfg_name]
    tokens = args.tokens or default_tokens

    if args.impl == "reference":
        run_reference_arm(args, cfg, tokens)
    elif args.gpus > 1 or int(os.environ.get("WORLD_SIZE", "1")) > 1:
        run_expert_parallel(args, cfg, tokens)
    else:
        run_single_gpu(args, cfg, tokens, bound)


if __name__ == "__main__":
    main()
