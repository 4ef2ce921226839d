"""The other forms an expert's weights may be resident in on the same node
(runtime-rs/shaders/independent_sparse_moe_gate_up_batch1_mxfp4.comp.template:166-228,250-355):
pre-expanded FP8 (address-record representation 1: the packaged E2M1 codes as E4M3 bytes, same
scales), chosen per expert at run time, and native FP8 resources (E4M3 weights with one E8M0 scale
per 128 x 128 block) for the ids from NATIVE_FP8_RESOURCE_START on.  Both expert paths, against the
CPU checker."""
import numpy as np
import pytest

from nerve_b200 import synthetic
from nerve_b200.backend import CudaComputeDevice, ExpertBank, MoePlan, geometry_from_config
from oracle import moe_oracle as mo
from tests.helpers import assert_close, expert_params, router_params

pytestmark = pytest.mark.gpu
PATHS = [pytest.param(1, id="simt"), pytest.param(2, id="tcgen05")]


@pytest.fixture(scope="module")
def device():
    dev = CudaComputeDevice(0)
    yield dev
    dev.close()


def run_layer(device, cfg, case, tokens, path, tensors, expanded=()):
    plan = MoePlan(device, geometry_from_config(cfg, tokens))
    plan.set_expert_path(path)
    bank = ExpertBank.upload(device, *tensors, expanded=set(expanded))
    hidden = device.resident_buffer_from(case.hidden)
    rw = device.resident_buffer_from(case.router_w)
    rbias = device.resident_buffer_from(case.router_bias) if case.router_bias is not None else None
    sbias = device.resident_buffer_from(case.select_bias) if case.select_bias is not None else None
    out = device.create_resident_buffer(tokens * cfg.hidden * 2)
    routes = device.create_resident_buffer(tokens * cfg.total_k * 4)
    plan.layer(tokens, bank, hidden, out, router_weights=rw, router_bias=rbias, bias=sbias, routes_out=routes)
    result = out.read(np.uint16).reshape(tokens, cfg.hidden), routes.read(np.uint32).reshape(tokens, cfg.total_k), plan.status()
    plan.destroy()
    bank.destroy()
    return result


def oracle_layer_with(cfg, case, weights, tier=1):
    logits = mo.linear_bf16(case.hidden, case.router_w, case.router_bias)
    out, routes, _, _ = mo.moe_layer(router_params(cfg), expert_params(cfg, tier), case.hidden, logits, case.select_bias, weights)
    return out, routes


@pytest.mark.parametrize("path", PATHS)
@pytest.mark.parametrize("hidden,intermediate,block", [(256, 384, 32), (512, 256, 128)])
def test_pre_expanded_experts_give_the_compact_result(device, path, hidden, intermediate, block):
    cfg = synthetic.MoeConfig("forms", hidden, intermediate, 8, 2, act_block=block, swiglu_limit=7.0)
    tokens = 90
    case = synthetic.make_case(cfg, tokens, seed=31)
    compact = (case.w1, case.s1, case.w3, case.s3, case.w2, case.s2)
    expanded = {1, 2, 5, 7}
    mixed = tuple([synthetic.expand_to_e4m3(t[e]) if (i % 2 == 0 and e in expanded) else t[e] for e in range(cfg.total_experts)]
                  for i, t in enumerate(compact))
    base, base_routes, status = run_layer(device, cfg, case, tokens, path, compact)
    assert status == 0
    got, got_routes, status = run_layer(device, cfg, case, tokens, path, mixed, expanded)
    assert status == 0
    np.testing.assert_array_equal(got_routes, base_routes)
    # the expanded bytes are the same values: the same products and sums, the same bits
    np.testing.assert_array_equal(got, base)
    want, want_routes = oracle_layer_with(cfg, case, mo.ExpertWeights(*mixed, expanded=frozenset(expanded)))
    np.testing.assert_array_equal(got_routes, want_routes)
    assert_close(got, want, f"pre-expanded experts {hidden}x{intermediate} path{path}")


@pytest.mark.parametrize("path", PATHS)
def test_a_pair_in_two_forms_fails_closed(device, path):
    cfg = synthetic.MoeConfig("forms", 256, 256, 4, 2, act_block=128)
    tokens = 16
    case = synthetic.make_case(cfg, tokens, seed=5)
    tensors = [list(t) for t in (case.w1, case.s1, case.w3, case.s3, case.w2, case.s2)]
    plan = MoePlan(device, geometry_from_config(cfg, tokens))
    plan.set_expert_path(path)
    # expert 2: w1 pre-expanded, w3 compact: the shader's gate_preexpanded == up_preexpanded rule rejects it
    tensors[0][2] = synthetic.expand_to_e4m3(tensors[0][2])
    bank = ExpertBank.upload(device, *tensors)
    words = bank.gate_up_addresses.read(np.uint32).copy()
    words[(2 * 4 + 0) * 8 + 7] = 1
    bank.gate_up_addresses.write_bytes(words)
    hidden = device.resident_buffer_from(case.hidden)
    rw = device.resident_buffer_from(case.router_w)
    out = device.create_resident_buffer(tokens * cfg.hidden * 2)
    routes = device.create_resident_buffer(tokens * cfg.total_k * 4)
    plan.layer(tokens, bank, hidden, out, router_weights=rw, routes_out=routes)
    assert plan.status() & 4, "routes to the inconsistent expert must be skipped with EXPERT_NOT_RESIDENT"
    # the checker skips the same routes
    weights = mo.ExpertWeights(*tensors)
    ga, gs = weights.gate_up_tables()
    ga[(2 * 4 + 0) * 8 + 7] = 1
    logits = mo.linear_bf16(case.hidden, case.router_w, None)
    got_routes = routes.read(np.uint32).reshape(tokens, cfg.total_k)
    ep = expert_params(cfg, 1)
    inter = np.zeros((tokens, ep.frame_words), dtype=np.uint32)
    control = np.array([tokens, 0, 0, 0, 0, 0, 0], dtype=np.uint32)
    mo.route_compact(got_routes, inter, control, cfg.intermediate, cfg.total_k, -(-cfg.intermediate // 32))
    mo.gate_up(ep, case.hidden, got_routes, inter, ga, gs, control)
    da, ds = weights.down_tables()
    outs = np.zeros((tokens, cfg.total_k, cfg.hidden), dtype=np.uint16)
    mo.down(ep, inter, got_routes, outs, da, ds, control)
    assert_close(out.read(np.uint16).reshape(tokens, cfg.hidden), mo.reduce(outs, tokens, cfg.total_k, cfg.hidden))
    plan.destroy()


@pytest.mark.parametrize("path", PATHS)
@pytest.mark.parametrize("tokens", [3, 200])
def test_native_fp8_shared_resource_beside_mxfp4_experts(device, path, tokens):
    """The DeepSeek-style layer: routed experts in packaged MXFP4, the always-selected shared expert as a native
    FP8 resource on the same node."""
    cfg = synthetic.small_variant(synthetic.CONFIGS["deepseek-v3"], 512, 256, 32)
    cfg = synthetic.replace(cfg, native_fp8_resources=1)
    case = synthetic.make_case(cfg, tokens, seed=9)
    tensors = [list(t) for t in (case.w1, case.s1, case.w3, case.s3, case.w2, case.s2)]
    for i, t in enumerate(synthetic.native_fp8_tensors(cfg, 9, cfg.experts)):
        tensors[i][cfg.experts] = t
    got, got_routes, status = run_layer(device, cfg, case, tokens, path, tensors)
    assert status == 0
    want, want_routes = oracle_layer_with(cfg, case, mo.ExpertWeights(*tensors))
    np.testing.assert_array_equal(got_routes, want_routes)
    assert_close(got, want, f"native FP8 shared resource T{tokens} path{path}")
    # the shared resource matters: without it the result differs
    assert (got_routes[:, -1] & 0xFFFF == cfg.experts).all()
