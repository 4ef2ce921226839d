"""MoE-layer benchmark: tokens/s of the route-native MXFP4 sparse-expert layer on B200.

    python bench.py --gpus N --steps K --warmup W [--workload NAME] [--tokens T] [--impl reference]

A step is one pass of the whole layer (router projection, routing, schedule, gate/up + SwiGLU,
down, combine) over one batch of seeded synthetic tokens.  `value` is timed with the inputs
resident in HBM (CUDA events on the launching stream, one pair per step, L2 flushed between
steps); `e2e` is the same metric through the host-buffer call, host<->device copies inside the
timed region.  The `roofline` object is for the dominant kernel (gate/up), the `cpu_baseline`
object times the CPU restatement of the reference shaders on this box's host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from nerve_b200 import synthetic  # noqa: E402

METRIC = "moe_layer_tokens_per_s"
UNIT = "tokens/s"
L2_BYTES = 126 * 1024 * 1024  # B200 L2

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


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines: list[str] = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, smax, reasons = [], None, set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                smax = float(parts[1])
            except ValueError:
                continue
            for name, flag in zip(names, parts[3:7]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": smax, "reasons": sorted(reasons),
                "samples": len(sm)}


def algorithmic_bytes(cfg: synthetic.MoeConfig, tokens: int, distinct: int) -> dict:
    """Bytes a perfect implementation moves per layer call (each selected expert's weights once)."""
    H, I = cfg.hidden, cfg.intermediate
    gate_up = distinct * 2 * H * I * 17 // 32 + tokens * H  # w1 + w3 codes and scales, quantised tokens
    down = distinct * H * I * 17 // 32 + tokens * cfg.total_k * I
    layer = distinct * cfg.expert_weight_bytes + 2 * tokens * H * 2 + cfg.experts * H * 2
    return {"gate_up": gate_up, "down": down, "layer": layer}


def layer_flops(cfg: synthetic.MoeConfig, tokens: int) -> float:
    return 2.0 * tokens * cfg.total_k * 3 * cfg.hidden * cfg.intermediate


class LayerRunner:
    """One rank's resident layer: weights, plan, device buffers."""

    def __init__(self, cfg, tokens, seed, expert_path, device_index=0, expert_start=0, expert_count=0, banks=0):
        from nerve_b200.backend import CudaComputeDevice, ExpertBank, MoePlan

        self.cfg, self.tokens = cfg, tokens
        self.device = CudaComputeDevice(device_index)
        self.case = synthetic.make_case(cfg, tokens, seed=seed, with_weights=False)
        # weights are generated and uploaded one expert at a time to keep host memory flat
        owned = range(cfg.total_experts) if not expert_count else range(expert_start, expert_start + expert_count)
        w = {k: [None] * cfg.total_experts for k in ("w1", "s1", "w3", "s3", "w2", "s2")}
        H, I = cfg.hidden, cfg.intermediate
        for e in owned:
            g = synthetic._stream(seed, f"expert{e}")
            w["w1"][e] = g.integers(0, 256, (I, H // 2), dtype=np.uint8)
            w["s1"][e] = g.integers(121, 128, (I, H // 32), dtype=np.uint8)
            w["w3"][e] = g.integers(0, 256, (I, H // 2), dtype=np.uint8)
            w["s3"][e] = g.integers(121, 128, (I, H // 32), dtype=np.uint8)
            w["w2"][e] = g.integers(0, 256, (H, I // 2), dtype=np.uint8)
            w["s2"][e] = g.integers(121, 128, (H, I // 32), dtype=np.uint8)
        # Several resident copies of the layer's weights ("banks", as a model's successive layers would be),
        # visited in turn: the weights a step reads were last read a whole cycle ago, and the cycle is
        # several times the L2 size, so every step streams its weights from HBM without dirtying L2 first.
        per_expert = 3 * H * I * 17 // 32
        touched = max(1, min(tokens * cfg.total_k, len(owned))) * per_expert
        self.n_banks = banks or max(2, min(8, -(-4 * L2_BYTES // touched)))
        self.banks = [ExpertBank.upload(self.device, w["w1"], w["s1"], w["w3"], w["s3"], w["w2"], w["s2"], present=list(owned))
                      for _ in range(self.n_banks)]
        self.bank = self.banks[0]
        self.cycle_bytes = touched * self.n_banks
        self.turn = 0
        self.host_weights = w if os.environ.get("NVMOE_BENCH_KEEP_WEIGHTS") else None
        self.plan = MoePlan.for_config(self.device, cfg, tokens)
        if expert_path:
            self.plan.set_expert_path(expert_path)
        self.plan.set_profiling(True)
        c = self.case
        self.hidden = self.device.resident_buffer_from(c.hidden)
        self.router_w = self.device.resident_buffer_from(c.router_w)
        self.router_bias = self.device.resident_buffer_from(c.router_bias) if c.router_bias is not None else None
        self.select_bias = self.device.resident_buffer_from(c.select_bias) if c.select_bias is not None else None
        self.output = self.device.create_resident_buffer(tokens * cfg.hidden * 2)
        self.telemetry = self.device.create_resident_buffer(self.plan.telemetry_words() * 4)
        # the end-to-end call reads its tokens from, and writes its result to, page-locked host memory
        import torch

        self._pinned = (torch.empty((tokens, cfg.hidden), dtype=torch.int16).pin_memory(),
                        torch.empty((tokens, cfg.hidden), dtype=torch.int16).pin_memory())
        self.hidden_host = self._pinned[0].numpy().view(np.uint16)
        self.hidden_host[...] = c.hidden
        self.out_host = self._pinned[1].numpy().view(np.uint16)
        self.kw = dict(router_weights=self.router_w, router_bias=self.router_bias, bias=self.select_bias,
                       telemetry=self.telemetry, expert_start=expert_start, expert_count=expert_count)

    def next_bank(self):
        self.turn += 1
        return self.banks[self.turn % self.n_banks]

    def step_resident(self) -> dict:
        self.plan.layer(self.tokens, self.next_bank(), self.hidden, self.output, **self.kw)
        return self.plan.last_report()

    def launch_step(self) -> None:
        """One layer call, nothing read back: the stream keeps running."""
        self.plan.layer(self.tokens, self.next_bank(), self.hidden, self.output, **self.kw)

    def step_host(self) -> float:
        bank = self.next_bank()
        t0 = time.perf_counter()
        self.plan.layer_host(self.tokens, bank, self.hidden_host, self.out_host, **self.kw)
        return (time.perf_counter() - t0) * 1e3


def flush_l2(torch, scratch):
    if scratch is None:
        return
    scratch.add_(1)  # read + write of a buffer larger than L2
    torch.cuda.synchronize()


def cpu_baseline(cfg, tokens, seed, sample_tokens, budget_s=12.0):
    """Times the CPU restatement of the reference shaders on a bounded sample of the workload: `sample_tokens`
    tokens first (a probe of the host's speed), then as many tokens of the workload as about `budget_s`
    seconds take, passed over repeatedly if the whole workload takes less."""
    from oracle import moe_oracle as mo

    probe = _cpu_layer_pass(cfg, tokens, seed, min(tokens, sample_tokens), passes=1)
    rate = probe["value"]
    sample = int(max(1, min(tokens, rate * budget_s)))
    passes = int(max(1, min(50, budget_s * rate / sample)))
    result = _cpu_layer_pass(cfg, tokens, seed, sample, passes)
    # one host core, on a sample a few per cent of that size
    threads = mo.lib().oracle_set_threads(1)
    try:
        few = int(max(1, min(tokens, rate * budget_s / (8.0 * max(1, threads)))))
        result["single_core_value"] = _cpu_layer_pass(cfg, tokens, seed, few, passes=1)["value"]
    finally:
        mo.lib().oracle_set_threads(threads)
    return result


def _cpu_layer_pass(cfg, tokens, seed, sample, passes):
    from oracle import moe_oracle as mo

    router_params, expert_params = mo.router_params_from, mo.expert_params_from
    case = synthetic.make_case(cfg, sample, seed=seed, with_weights=False)
    logits = mo.linear_bf16(case.hidden, case.router_w, case.router_bias)
    routes, _ = mo.route(router_params(cfg), logits, case.select_bias)
    used = sorted(set((routes.reshape(-1) & 0xFFFF).tolist()))
    full = case
    H, I = cfg.hidden, cfg.intermediate
    empty = np.zeros((1, 1), dtype=np.uint8)
    w = {k: [empty] * cfg.total_experts for k in ("w1", "s1", "w3", "s3", "w2", "s2")}
    for e in used:
        g = synthetic._stream(seed, f"expert{e}")
        w["w1"][e] = g.integers(0, 256, (I, H // 2), dtype=np.uint8)
        w["s1"][e] = g.integers(121, 128, (I, H // 32), dtype=np.uint8)
        w["w3"][e] = g.integers(0, 256, (I, H // 2), dtype=np.uint8)
        w["s3"][e] = g.integers(121, 128, (I, H // 32), dtype=np.uint8)
        w["w2"][e] = g.integers(0, 256, (H, I // 2), dtype=np.uint8)
        w["s2"][e] = g.integers(121, 128, (H, I // 32), dtype=np.uint8)
    weights = mo.ExpertWeights(w["w1"], w["s1"], w["w3"], w["s3"], w["w2"], w["s2"])
    rp, ep = router_params(cfg), expert_params(cfg, tier=0)  # tier 0: the shaders' f32 accumulation order
    t0 = time.perf_counter()
    for _ in range(passes):
        logits = mo.linear_bf16(full.hidden, full.router_w, full.router_bias)
        mo.moe_layer(rp, ep, full.hidden, logits, full.select_bias, weights)
    seconds = time.perf_counter() - t0
    return {"value": passes * sample / seconds, "unit": UNIT, "cores": mo.lib().oracle_max_threads(), "kind": "port",
            "sample": f"{sample} of {tokens} tokens, whole layer, {passes} pass(es), {seconds:.2f} s",
            "sample_tokens": sample}


def run_reference_arm(args, cfg, tokens):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    sample_tokens = max(1, min(tokens, args.reference_sample))
    values = []
    budget = min(10.0, 120.0 / max(1, args.warmup + args.steps))  # the whole run stays within a few minutes
    for _ in range(args.warmup + args.steps):
        values.append(cpu_baseline(cfg, tokens, args.seed, sample_tokens, budget_s=budget))
    timed = values[args.warmup:] or values
    value = statistics.mean(v["value"] for v in timed)
    base = dict(timed[-1])
    base["value"] = value
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1e3 * base["sample_tokens"] / value, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "fp8_e4m3 x mxfp4_e2m1 -> f32", "data": "synthetic",
        "config": {"workload": args.workload, "tokens": tokens, "hidden": cfg.hidden, "intermediate": cfg.intermediate,
                   "experts": cfg.experts, "k": cfg.total_k,
                   "note": "CPU restatement of the reference shaders (the reference has no CPU backend); each step is a bounded token sample of the workload"},
        "cpu_baseline": base,
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


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
    ap.add_argument("--reference-sample", type=int, default=16, help="tokens per step of the CPU arm")
    ap.add_argument("--no-extra", action="store_true", help="skip the additional batch sizes")
    ap.add_argument("--l2", default="rotate", choices=["rotate", "flush"],
                    help="rotate: inputs larger than L2 (weight banks visited in turn); flush: also rewrite a 256 MB buffer between steps")
    ap.add_argument("--banks", type=int, default=0, help="resident weight copies visited in turn (0 = enough for 4 x L2 per cycle)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "native" else args.warmup

    cfg_name, default_tokens, bound = WORKLOADS[args.workload]
    cfg = synthetic.CONFIGS[cfg_name]
    tokens = args.tokens or default_tokens

    if args.impl == "reference":
        run_reference_arm(args, cfg, tokens)
        return

    if args.gpus > 1 or int(os.environ.get("WORLD_SIZE", "1")) > 1:
        from nerve_b200 import expert_parallel

        expert_parallel.bench_main(args, cfg, tokens, METRIC, UNIT)
        return

    import torch

    torch.cuda.init()
    peaks, peak_kind = measured_peaks()
    runner = LayerRunner(cfg, tokens, args.seed, args.expert_path, banks=args.banks)
    # --l2 flush: additionally rewrite a 256 MB buffer between timed steps (leaves L2 full of dirty lines
    # whose write-back then competes with the step's reads); default: the rotating weight banks alone
    scratch = torch.empty(256 * 1024 * 1024 // 4, dtype=torch.int32, device="cuda:0") if args.l2 == "flush" else None

    def timed_steps(r, steps, warmup, sample_clocks=False):
        for _ in range(max(warmup, r.n_banks + 1)):  # every bank's tables are resolved once before timing
            r.step_resident()
            r.device.synchronize()
        sampler = ClockSampler(0) if sample_clocks else None
        if sampler:
            sampler.start()
        reports = []
        for _ in range(steps):
            flush_l2(torch, scratch)
            reports.append(r.step_resident())  # last_report synchronises the stream
        clocks = sampler.stop() if sampler else None
        return reports, clocks

    def timed_block(r, steps, warmup, sample_clocks=False):
        """The contract's timed region: exactly `steps` layer calls back to back between two CUDA events on
        the stream they run on, a synchronise on both sides, no per-stage events inside."""
        r.plan.set_profiling(False)
        stream = torch.cuda.ExternalStream(r.device.stream(), device="cuda:0")
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for _ in range(max(warmup, r.n_banks + 1)):
            r.launch_step()
        torch.cuda.synchronize()
        sampler = ClockSampler(0) if sample_clocks else None
        if sampler:
            sampler.start()
        if scratch is not None:
            flush_l2(torch, scratch)
        before = r.plan.launches()
        begin.record(stream)
        for _ in range(steps):
            r.launch_step()
        end.record(stream)
        torch.cuda.synchronize()
        clocks = sampler.stop() if sampler else None
        r.plan.set_profiling(True)
        return begin.elapsed_time(end) / steps, r.plan.launches() - before, clocks

    # whole-layer throughput first (no profiling events in the stream), then per-kernel times from a
    # second pass with an event pair around each stage and each expert kernel
    ms, launches, clocks = timed_block(runner, args.steps, args.warmup, sample_clocks=True)
    reports, _ = timed_steps(runner, args.steps, args.warmup)
    profiled_ms = statistics.mean(rep["total_ms"] for rep in reports)
    gate_ms = statistics.mean(rep["gate_up_kernel_ms"] for rep in reports)
    down_ms = statistics.mean(rep["down_kernel_ms"] for rep in reports)
    distinct = reports[-1]["distinct_experts"]
    value = tokens / (ms * 1e-3)

    # end to end: host buffers in and out, copies inside the timed region
    runner.plan.set_profiling(False)
    for _ in range(max(3, runner.n_banks + 1)):
        runner.step_host()
    e2e_ms = []
    for _ in range(args.steps):
        flush_l2(torch, scratch)
        e2e_ms.append(runner.step_host())
    e2e_value = tokens / (statistics.mean(e2e_ms) * 1e-3)

    ab = algorithmic_bytes(cfg, tokens, distinct)
    # dram__bytes_read.sum + dram__bytes_write.sum of one launch, from the ncu capture summarised under
    # profiles/ (taken on this workload); other workloads have no capture and report null
    ncu_traffic = {("gpt-oss-20b-decode", 64): {"gate_up": 289069568, "down": 146978816}}.get((args.workload, tokens))
    if bound == "hbm":
        achieved = ab["gate_up"] / (gate_ms * 1e-3) / 1e9
        roofline = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                    "frac": achieved / peaks["hbm_gbs"], "traffic": ncu_traffic["gate_up"] if ncu_traffic else None,
                    "kernel": "gate_up",
                    "peak_kind": f"{peak_kind} STREAM-style copy",
                    "algorithmic_bytes_per_launch": ab["gate_up"], "kernel_ms": gate_ms,
                    "down_kernel": {"achieved": ab["down"] / (down_ms * 1e-3) / 1e9, "kernel_ms": down_ms,
                                    "frac": ab["down"] / (down_ms * 1e-3) / 1e9 / peaks["hbm_gbs"]},
                    "layer": {"achieved": ab["layer"] / (ms * 1e-3) / 1e9, "frac": ab["layer"] / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"]}}
    else:
        flops_gate = 2.0 * tokens * cfg.total_k * 2 * cfg.hidden * cfg.intermediate
        achieved = flops_gate / (gate_ms * 1e-3) / 1e12
        peak = peaks["bf16_tflops"] * 2.0  # FP8-rate kinds run at twice the measured bf16 rate
        roofline = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                    "traffic": None, "kernel": "gate_up", "mma_kind": "mxf8f6f4 (E4M3 activations x E2M1 weights)",
                    "peak_kind": f"2 x {peak_kind} cuBLAS bf16 burst rate; against the mxf4 rate (4 x bf16) the fraction halves",
                    "kernel_ms": gate_ms, "frac_of_mxf4_rate": achieved / (peaks["bf16_tflops"] * 4.0),
                    "down_kernel": {"achieved": flops_gate / 2.0 / (down_ms * 1e-3) / 1e12, "kernel_ms": down_ms,
                                    "frac": flops_gate / 2.0 / (down_ms * 1e-3) / 1e12 / peak},
                    "layer": {"achieved": layer_flops(cfg, tokens) / (ms * 1e-3) / 1e12,
                              "frac": layer_flops(cfg, tokens) / (ms * 1e-3) / 1e12 / peak}}

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "fp8_e4m3 x mxfp4_e2m1 -> f32", "data": "synthetic",
        "config": {"workload": args.workload, "tokens": tokens, "hidden": cfg.hidden, "intermediate": cfg.intermediate,
                   "experts": cfg.experts, "k": cfg.total_k, "distinct_experts": distinct,
                   "expert_path": "tcgen05" if reports[-1]["tensor_path"] else "cuda-cores",
                   "l2": (f"inputs larger than L2: {runner.n_banks} resident weight banks visited in turn, "
                          f"{runner.cycle_bytes / 1e6:.0f} MB of weights read between two reads of the same bytes"
                          + ("; plus a 256 MB buffer rewritten between timed steps" if args.l2 == "flush" else "")),
                   "parallelism": "single device"},
        "clocks": clocks, "roofline": roofline,
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": tokens * cfg.hidden * 2,
                "d2h_bytes_per_step": tokens * cfg.hidden * 2, "ms_per_step": statistics.mean(e2e_ms)},
        "gpu_launches": launches,
        "stage_ms": {k: statistics.mean(rep["stage_ms"][k] for rep in reports) for k in reports[-1]["stage_ms"]},
        "profiled_ms_per_step": profiled_ms,
    }

    if not args.no_extra and args.workload == "gpt-oss-20b-decode":
        extra = {}
        for t in (1, 8, 32):
            r = LayerRunner(cfg, t, args.seed, args.expert_path, banks=args.banks)
            t_ms, _, _ = timed_block(r, max(5, args.steps // 2), 3)
            reps, _ = timed_steps(r, max(5, args.steps // 2), 3)
            d = reps[-1]["distinct_experts"]
            b = algorithmic_bytes(cfg, t, d)
            extra[f"decode_T{t}"] = {"tokens_per_s": t / (t_ms * 1e-3), "ms_per_step": t_ms, "distinct_experts": d,
                                     "layer_hbm_frac": b["layer"] / (t_ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                                     "gate_up_hbm_frac": b["gate_up"] / (statistics.mean(x["gate_up_kernel_ms"] for x in reps) * 1e-3) / 1e9 / peaks["hbm_gbs"]}
        line["extra"] = extra

    if not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(cfg, tokens, args.seed, args.reference_sample)
    print(json.dumps(line))


if __name__ == "__main__":
    main()
