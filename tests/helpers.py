"""Shared plumbing of the parity tests: one synthetic case on the device and in the checker."""
from __future__ import annotations

import numpy as np

from nerve_b200 import synthetic
from oracle import moe_oracle as mo


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


def error_metrics(got_bf16: np.ndarray, want_bf16: np.ndarray) -> dict:
    g = mo.bf16_to_f32(got_bf16).astype(np.float64).reshape(-1)
    w = mo.bf16_to_f32(want_bf16).astype(np.float64).reshape(-1)
    diff = np.abs(g - w)
    scale = max(np.abs(w).max(), 1e-30)
    return {
        "max_abs": float(diff.max()),
        "max_abs_over_peak": float(diff.max() / scale),
        "rel_l2": float(np.sqrt((diff ** 2).sum()) / max(np.sqrt((w ** 2).sum()), 1e-30)),
        "mismatched": int((got_bf16.reshape(-1) != want_bf16.reshape(-1)).sum()),
        "count": int(w.size),
    }


# north_star tolerance for bf16 outputs against the f64-accumulated dequantised reference on the
# same quantised operands: rel-L2 <= 5e-3 and max-abs <= 2e-2 of the output's peak magnitude
REL_L2_TOL = 5e-3
MAX_ABS_TOL = 2e-2


def assert_close(got_bf16, want_bf16, what=""):
    m = error_metrics(got_bf16, want_bf16)
    assert m["rel_l2"] <= REL_L2_TOL and m["max_abs_over_peak"] <= MAX_ABS_TOL, (what, m)
    return m
