"""GPU parity at the full sizes of the benchmark configs, through the C ABI.

The counterpart of the reference's "real geometry" conformance run
(runtime-rs/src/vulkan_compute/mxfp4_tests.rs:316-1081): every shape the benchmark times is also
checked.  Logits, routes and the selection telemetry are compared bit for bit over the whole batch;
the layer output is compared with the CPU checker (tier 1: f64 accumulation on the operands the
kernels consume) on a seeded sample of tokens, which is exact in what it covers because a token's
output depends on nothing but its own row, its own routes and the weights of the experts they name.
"""
import numpy as np
import pytest

from nerve_b200 import synthetic
from nerve_b200.resident_layer import LayerRunner
from oracle import sampled
from tests.helpers import record_metrics

pytestmark = pytest.mark.gpu

# config name, batch sizes sharing one upload of the weights, sampled tokens per batch, expert paths
FULL_CASES = [
    pytest.param("gpt-oss-20b", (1, 8, 32, 64), 64, (1, 2), id="gpt-oss-20b-decode"),       # BASELINE configs[1]
    pytest.param("gpt-oss-20b-prefill", (4096,), 48, (1, 2), id="gpt-oss-20b-prefill-zipf"),  # configs[2]
    pytest.param("gpt-oss-120b", (8192,), 32, (2,), id="gpt-oss-120b"),                      # configs[3]
    pytest.param("deepseek-v3", (16384,), 16, (2,), id="deepseek-v3"),                       # configs[4]
]


def check_runner(runner: LayerRunner, sample_count: int, what: str) -> dict:
    """One layer call of `runner` against the checker; returns the error metrics of the sampled outputs."""
    cfg, case, tokens = runner.cfg, runner.case, runner.tokens
    logits_buf = runner.device.create_resident_buffer(tokens * ((cfg.experts + 1) // 2) * 4)
    runner.telemetry.fill(0)
    runner.plan.layer(tokens, runner.bank, runner.hidden, runner.output, logits=logits_buf, **runner.kw)
    assert runner.plan.status() == 0, "a kernel raised a fail-closed status bit"
    want_logits, want_routes, want_telemetry = sampled.routing_for_batch(cfg, case.hidden, case.router_w, case.router_bias,
                                                                         case.select_bias)
    np.testing.assert_array_equal(logits_buf.read(np.uint32).reshape(want_logits.shape), want_logits)
    np.testing.assert_array_equal(runner.read_routes(), want_routes)
    np.testing.assert_array_equal(runner.telemetry.read(np.uint32), want_telemetry)
    logits_buf.destroy()
    picked = sampled.sample_tokens(tokens, sample_count, seed=tokens)
    want = sampled.layer_on_sample(cfg, case.hidden, want_logits, case.select_bias, picked,
                                   lambda e: synthetic.expert_tensors(cfg, runner.seed, e))
    got = runner.read_output()[picked]
    metrics = sampled.error_metrics(got, want["output"])
    metrics["sample_tokens"] = int(len(picked))
    record_metrics(what, metrics)
    assert sampled.within_tolerance(metrics), (what, metrics)
    return metrics


@pytest.mark.parametrize("name,batches,sample_count,paths", FULL_CASES)
def test_full_size_layer_matches_checker(name, batches, sample_count, paths):
    cfg = synthetic.CONFIGS[name]
    first = None
    try:
        for path in paths:
            for tokens in batches:
                runner = LayerRunner(cfg, tokens, 0, path, banks=1, share=first)
                first = first or runner
                m = check_runner(runner, sample_count, f"{name} T{tokens} path{path} full size")
                print(f"\n{name} T{tokens} path {path}: routes, logits, telemetry bit-exact; {m}")
                if runner is not first:
                    runner.release()
    finally:
        if first is not None:
            first.release()
            for bank in first.banks:
                bank.destroy()
            first.device.close()
