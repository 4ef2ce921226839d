"""Shared plumbing of the parity tests: one synthetic case on the device and in the checker."""
from __future__ import annotations

import json
from pathlib import Path

import numpy as np

from nerve_b200 import synthetic
from oracle import moe_oracle as mo
from oracle import sampled


router_params = mo.router_params_from
expert_params = mo.expert_params_from


def oracle_weights(case: synthetic.MoeCase) -> mo.ExpertWeights:
    return mo.ExpertWeights(case.w1, case.s1, case.w3, case.s3, case.w2, case.s2)


def oracle_layer(case: synthetic.MoeCase, tier: int = 1, expert_start: int = 0, expert_count: int = 0):
    """logits by the checker's projection, then the whole node chain on the CPU."""
    cfg = case.cfg
    logits = mo.linear_bf16(case.hidden, case.router_w, case.router_bias)
    out, routes, outputs, inter = mo.moe_layer(
        router_params(cfg), expert_params(cfg, tier), case.hidden, logits, case.select_bias,
        oracle_weights(case), expert_start, expert_count)
    return {"logits": logits, "output": out, "routes": routes, "expert_outputs": outputs, "intermediates": inter}


error_metrics = sampled.error_metrics

# north_star tolerance for bf16 outputs against the f64-accumulated dequantised reference on the
# same quantised operands: rel-L2 <= 5e-3 and max-abs <= 2e-2 of the output's peak magnitude (the
# absolute max-abs is recorded beside it; see oracle/sampled.py for why the relative reading is gated)
REL_L2_TOL = sampled.REL_L2_TOL
MAX_ABS_TOL = sampled.MAX_ABS_OVER_PEAK_TOL


def assert_close(got_bf16, want_bf16, what=""):
    m = error_metrics(got_bf16, want_bf16)
    assert sampled.within_tolerance(m), (what, m)
    if what:
        record_metrics(what, m)
    return m


def record_metrics(case_id: str, metrics: dict) -> None:
    """Appends the measured error of one parity case to parity_metrics.jsonl in the run-output folder at the
    repository root, so that the figures behind a green run can be kept (profiles/ holds a summary)."""
    folder = Path(__file__).resolve().parent.parent / "gpurun_out"
    try:
        folder.mkdir(exist_ok=True)
        with open(folder / "parity_metrics.jsonl", "a") as f:
            f.write(json.dumps({"case": case_id, **metrics}) + "\n")
    except OSError:
        pass
