"""GPU parity of the expert projections, the combine and the whole layer, through the C ABI.

Known answers first (the reference's own constant-fill conformance cases), then seeded random
layers against the CPU checker: indices bit-exact, bf16 outputs within the stated tolerance of the
f64-accumulated reference on the same quantised operands.  Every case runs on both expert paths
(1 = CUDA-core dequant-GEMV, 2 = tcgen05 grouped MMA).
"""
import json
from pathlib import Path

import numpy as np
import pytest

from nerve_b200 import synthetic
from nerve_b200.backend import CudaComputeDevice, CudaError, ExpertBank, MoePlan, ResidentBuffer, address_table, geometry_from_config
from oracle import moe_oracle as mo
from tests.helpers import assert_close, error_metrics, expert_params, oracle_layer, oracle_weights, router_params

pytestmark = pytest.mark.gpu

GOLDEN = json.loads((Path(__file__).parent / "golden" / "reference_vectors.json").read_text())
PATHS = [pytest.param(1, id="simt"), pytest.param(2, id="tcgen05")]


@pytest.fixture(scope="module")
def device():
    dev = CudaComputeDevice(0)
    yield dev
    dev.close()


def make_plan(device, cfg, tokens, path):
    plan = MoePlan(device, geometry_from_config(cfg, tokens))
    try:
        plan.set_expert_path(path)
    except CudaError as error:
        plan.destroy()
        if error.code == -5:
            pytest.skip(f"expert path {path} does not take this geometry: {error.message}")
        raise
    return plan


BF16_ONE = 0x3F80


def _const_cfg(width, experts=1, k=1, limit=10.0):
    return synthetic.MoeConfig("const", width, width, experts, k, swiglu_limit=limit, act_block=128)


@pytest.mark.parametrize("path", PATHS)
def test_constant_fill_known_answers(device, path):
    """mxfp4_tests.rs:89-215 — hidden 1.0, weights 0x22 (=1.0), scales 120 (=2^-7): 128 columns sum
    to 1.0, so gate/up gives bf16(silu(1)) everywhere and down gives the E2M1 value of the nibble."""
    ka = GOLDEN["rust_known_answers"]["constant_fill"]
    W = ka["width"]
    cfg = _const_cfg(W, limit=ka["swiglu_limit"])
    plan = make_plan(device, cfg, 1, path)
    hidden = device.resident_buffer_from(np.full(W, BF16_ONE, dtype=np.uint16))
    routes = device.resident_buffer_from(np.array([BF16_ONE << 16], dtype=np.uint32))
    inter = device.create_resident_buffer(plan.frame_words * 4)
    wt = device.resident_buffer_from(np.full(W * W // 2, ka["weight_fill"], dtype=np.uint8))
    sc = device.resident_buffer_from(np.full(W * W // 32, ka["scale_fill"], dtype=np.uint8))
    gaddr = address_table(device, [wt, sc, wt, sc])
    gslots = device.resident_buffer_from(np.array([0, 1, 2, 3], dtype=np.uint32))
    control = device.resident_buffer_from(np.array([1, 0, 0, 0, 4, 1, 1], dtype=np.uint32))
    plan.independent_sparse_moe_gate_up(1, hidden, routes, inter, gaddr, gslots, control)
    expected = int(synthetic.f32_to_bf16(np.array([1.0 / (1.0 + np.exp(np.float32(-1.0)))], dtype=np.float32))[0])
    data = inter.read(np.uint16, W)
    assert np.all(data == expected), (data[:8], hex(expected))

    # the prequantised twin (0x38 = 1.0, scale 1.0) runs on the general path in every build
    inter.fill(0)
    qh = device.resident_buffer_from(np.full(W, ka["prequant_hidden_byte"], dtype=np.uint8))
    hs = device.resident_buffer_from(np.array([ka["prequant_scale"]], dtype=np.float32))
    plan.independent_sparse_moe_gate_up_prequant(1, qh, hs, routes, inter, gaddr, gslots, control)
    assert np.all(inter.read(np.uint16, W) == expected)

    inter.fill(0)
    inter.write_bytes(np.full(W, BF16_ONE, dtype=np.uint16))
    outputs = device.create_resident_buffer(W * 2)
    dwt = device.resident_buffer_from(np.full(W * W // 2, ka["weight_fill"], dtype=np.uint8))
    daddr = address_table(device, [dwt, sc])
    dslots = device.resident_buffer_from(np.array([0, 1], dtype=np.uint32))
    dcontrol = device.resident_buffer_from(np.array([1, 0, 0, 0, 2, 1, 1], dtype=np.uint32))
    plan.independent_sparse_moe_down(1, inter, routes, outputs, daddr, dslots, dcontrol)
    assert np.all(outputs.read(np.uint16) == BF16_ONE)
    for nibble, value in enumerate(ka["e2m1_values"]):
        dwt.write_bytes(np.full(W * W // 2, nibble | (nibble << 4), dtype=np.uint8))
        outputs.fill(0)
        plan.independent_sparse_moe_down(1, inter, routes, outputs, daddr, dslots, dcontrol)
        got = mo.bf16_to_f32(outputs.read(np.uint16))
        assert np.all(got == np.float32(value)), (nibble, got[:4])
    assert plan.status() == 0
    plan.destroy()


@pytest.mark.parametrize("path", PATHS)
def test_fails_closed_on_invalid_dynamic_metadata(device, path):
    """mxfp4_tests.rs:279-313 — an out-of-range compact route or an unpublished address record
    leaves the output untouched; so do the other record checks of the shader."""
    W = 128
    cfg = _const_cfg(W)
    plan = make_plan(device, cfg, 1, path)
    hidden = device.resident_buffer_from(np.full(W, BF16_ONE, dtype=np.uint16))
    routes = device.resident_buffer_from(np.array([BF16_ONE << 16], dtype=np.uint32))
    inter = device.create_resident_buffer(plan.frame_words * 4)
    wt = device.resident_buffer_from(np.full(W * W // 2, 0x22, dtype=np.uint8))
    sc = device.resident_buffer_from(np.full(W * W // 32, 120, dtype=np.uint8))
    gaddr = address_table(device, [wt, sc, wt, sc])
    good = gaddr.read(np.uint32).copy()
    gslots = device.resident_buffer_from(np.array([0, 1, 2, 3], dtype=np.uint32))
    control = device.resident_buffer_from(np.array([1, 0, 0, 0, 0, 0, 0], dtype=np.uint32))

    def run():
        plan.independent_sparse_moe_gate_up(1, hidden, routes, inter, gaddr, gslots, control)
        return inter.read(np.uint16, W)

    assert run().all()
    assert plan.status() == 0
    inter.fill(0)
    inter.write_bytes(np.array([0xFFFFFFFF], dtype=np.uint32), offset=plan.data_words * 4)
    assert not run().any()
    assert plan.status() & 2
    inter.write_bytes(np.array([0], dtype=np.uint32), offset=plan.data_words * 4)
    gaddr.write_bytes(np.zeros_like(good))
    assert not run().any()
    assert plan.status() & 4
    for word, value in ((4, 0), (6, 0), (6, 2), (2, 16), (0, int(good[0]) | 4), (7, 1)):
        broken = good.copy()
        broken[16 + word] = value  # third record: w3
        if word == 4:
            broken[16 + 5] = 0
        gaddr.write_bytes(broken)
        assert not run().any(), (word, value)
    gaddr.write_bytes(good)
    gslots.write_bytes(np.array([0, 1, 0xFFFFFFFF, 3], dtype=np.uint32))
    assert not run().any()
    gslots.write_bytes(np.array([0, 1, 2, 3], dtype=np.uint32))
    # an expert id beyond the resource count
    routes.write_bytes(np.array([(BF16_ONE << 16) | 5], dtype=np.uint32))
    assert not run().any()
    routes.write_bytes(np.array([BF16_ONE << 16], dtype=np.uint32))
    plan.status()
    assert run().all()
    plan.destroy()


@pytest.mark.parametrize("path", PATHS)
def test_table_changed_behind_its_handle_is_resolved_again_once_marked(device, path):
    """A slot table rewritten through its device address (here: through a second handle over the same
    memory) is only seen by a plan after nvmoe_buffer_mark_dirty; handles that wrap the same memory share
    one place in the plan's cache."""
    W = 128
    cfg = _const_cfg(W)
    plan = make_plan(device, cfg, 1, path)
    hidden = device.resident_buffer_from(np.full(W, BF16_ONE, dtype=np.uint16))
    routes = device.resident_buffer_from(np.array([BF16_ONE << 16], dtype=np.uint32))
    inter = device.create_resident_buffer(plan.frame_words * 4)
    wt = device.resident_buffer_from(np.full(W * W // 2, 0x22, dtype=np.uint8))
    sc = device.resident_buffer_from(np.full(W * W // 32, 120, dtype=np.uint8))
    gaddr = address_table(device, [wt, sc, wt, sc])
    gslots = device.resident_buffer_from(np.array([0, 1, 2, 3], dtype=np.uint32))
    control = device.resident_buffer_from(np.array([1, 0, 0, 0, 0, 0, 0], dtype=np.uint32))

    def run(slots):
        inter.fill(0)
        inter.write_bytes(np.array([0], dtype=np.uint32), offset=plan.data_words * 4)
        plan.independent_sparse_moe_gate_up(1, hidden, routes, inter, gaddr, slots, control)
        return inter.read(np.uint16, W)

    assert run(gslots).all()
    alias = ResidentBuffer.wrap(device, gslots.device_address(), 16)
    alias.write_bytes(np.array([0, 1, 0xFFFFFFFF, 3], dtype=np.uint32))  # unbinds w3 behind gslots' back
    assert run(gslots).all(), "the resolution kept for an unchanged handle is still in use"
    gslots.mark_dirty()
    assert not run(gslots).any()
    assert plan.status() & 4
    # tables in wrapped buffers are resolved on every call, whichever handle over the memory is passed
    alias.write_bytes(np.array([0, 1, 2, 3], dtype=np.uint32))
    assert run(alias).all()
    again = ResidentBuffer.wrap(device, gslots.device_address(), 16)
    assert run(again).all()
    for handle in (alias, again):
        handle.destroy()
    plan.destroy()


@pytest.mark.parametrize("path", PATHS)
def test_route_native_matches_canonical_bit_exactly(device, path):
    """mxfp4_route_native_tests.rs:7-250 — routes {3:0.75, 1:0.25}, only experts 1 and 3 bound:
    scheduler + partitioned projection == canonical projection, control words as published."""
    ka = GOLDEN["rust_known_answers"]["route_native"]
    H, I, E, K = ka["hidden"], ka["intermediate"], ka["experts"], ka["k"]
    cfg = synthetic.MoeConfig("rn", H, I, E, K, swiglu_limit=10.0, act_block=128)
    plan = make_plan(device, cfg, 1, path)
    route_words = np.array([e | (int(synthetic.f32_to_bf16(np.array([w], dtype=np.float32))[0]) << 16)
                            for e, w in ka["routes"]], dtype=np.uint32)
    routes = device.resident_buffer_from(route_words)
    hidden = device.resident_buffer_from(np.full(H, BF16_ONE, dtype=np.uint16))
    fills = {int(e): v for e, v in ka["fills"].items()}
    n = E
    w1 = [np.full((I, H // 2), fills.get(e, 0), dtype=np.uint8) for e in range(n)]
    s1 = [np.full((I, H // 32), ka["scale_fill"], dtype=np.uint8) for e in range(n)]
    w2 = [np.full((H, I // 2), fills.get(e, 0), dtype=np.uint8) for e in range(n)]
    s2 = [np.full((H, I // 32), ka["scale_fill"], dtype=np.uint8) for e in range(n)]
    bank = ExpertBank.upload(device, w1, s1, w1, s1, w2, s2, present=ka["bound_experts"])
    inter = device.create_resident_buffer(plan.frame_words * 4)
    outputs = device.create_resident_buffer(K * H * 2)

    def reset():
        words = np.zeros(plan.frame_words, dtype=np.uint32)
        words[plan.data_words:] = np.arange(K)
        inter.write_bytes(words)
        outputs.fill(0)

    reset()
    gc = device.resident_buffer_from(np.array(ka["canonical_control"]["gate"], dtype=np.uint32))
    dc = device.resident_buffer_from(np.array(ka["canonical_control"]["down"], dtype=np.uint32))
    plan.independent_sparse_moe_gate_up(1, hidden, routes, inter, bank.gate_up_addresses, bank.gate_up_slots, gc)
    plan.independent_sparse_moe_down(1, inter, routes, outputs, bank.down_addresses, bank.down_slots, dc)
    canonical = outputs.read(np.uint16).copy()
    assert canonical.any()

    reset()
    gc.write_bytes(np.array(ka["control_in"], dtype=np.uint32))
    dc.write_bytes(np.array(ka["control_in"], dtype=np.uint32))
    plan.moe_route_compact(1, routes, inter, gc)
    plan.independent_sparse_moe_gate_up(1, hidden, routes, inter, bank.gate_up_addresses, bank.gate_up_slots, gc)
    plan.moe_route_count(1, routes, dc)
    plan.independent_sparse_moe_down(1, inter, routes, outputs, bank.down_addresses, bank.down_slots, dc)
    assert gc.read(np.uint32).tolist() == ka["gate_control_out"]
    assert dc.read(np.uint32).tolist() == ka["down_control_out"]
    np.testing.assert_array_equal(outputs.read(np.uint16), canonical)
    # and both equal the checker
    want = np.zeros((1, K, H), dtype=np.uint16)
    oi = np.zeros((1, plan.frame_words), dtype=np.uint32)
    oi[0, plan.data_words:] = np.arange(K)
    ow = mo.ExpertWeights(w1, s1, w1, s1, w2, s2)
    ga, gs = ow.gate_up_tables(ka["bound_experts"])
    da, ds = ow.down_tables(ka["bound_experts"])
    ep = expert_params(cfg, tier=1)
    oc = np.array(ka["canonical_control"]["gate"], dtype=np.uint32)
    mo.gate_up(ep, np.full((1, H), BF16_ONE, dtype=np.uint16), route_words[None, :], oi, ga, gs, oc)
    mo.down(ep, oi, route_words[None, :], want, da, ds, np.array(ka["canonical_control"]["down"], dtype=np.uint32))
    np.testing.assert_array_equal(canonical, want.reshape(-1))
    plan.destroy()


def test_reduce_is_bit_exact(device):
    rng = np.random.default_rng(5)
    T, K, H = 37, 9, 256
    x = synthetic.f32_to_bf16(rng.standard_normal((T, K, H), dtype=np.float32) * 3)
    cfg = synthetic.MoeConfig("r", H, 128, 16, K)
    g = geometry_from_config(cfg, T)
    g.reduce_scale = 2.5
    plan = MoePlan(device, g)
    xb = device.resident_buffer_from(x)
    ob = device.create_resident_buffer(T * H * 2)
    plan.moe_reduce(T, xb, ob)
    np.testing.assert_array_equal(ob.read(np.uint16).reshape(T, H), mo.reduce(x, T, K, H, 2.5))
    plan.destroy()


LAYER_CASES = [
    pytest.param("tiny", None, 64, id="tiny-T64"),                                  # BASELINE configs[0]
    pytest.param("gpt-oss-20b", (256, 384, 16), 1, id="gptoss-small-T1"),
    pytest.param("gpt-oss-20b", (256, 384, 16), 33, id="gptoss-small-T33"),
    pytest.param("gpt-oss-20b", (2880, 2880, 32), 8, id="gptoss-20b-T8"),            # configs[1] shape
    pytest.param("gpt-oss-20b-prefill", (352, 160, 32), 600, id="gptoss-zipf-small-T600"),
    # wide token tiles on the TMA path: ragged row tiles (320 = 2.5 x 128), a K tail in down, row pairs with a lone half
    pytest.param("gpt-oss-20b-prefill", (384, 320, 8), 300, id="gptoss-zipf-tma-T300"),
    pytest.param("deepseek-v3", (512, 256, 32), 50, id="deepseek-small-T50"),
    pytest.param("deepseek-v3", (7168, 2048, 16), 4, id="deepseek-wide-T4"),
]


_CASE_CACHE = {}


def _case_and_reference(name, small, tokens):
    """The case, the same-operand reference (tier 1) and the unquantised-activation one (tier 2),
    computed once and shared by both expert paths."""
    key = (name, small, tokens)
    if key not in _CASE_CACHE:
        _CASE_CACHE.clear()  # one case at a time: the big ones hold hundreds of MB
        cfg = synthetic.CONFIGS[name]
        if small:
            cfg = synthetic.small_variant(cfg, *small)
        case = synthetic.make_case(cfg, tokens, seed=0)
        _CASE_CACHE[key] = (cfg, case, oracle_layer(case, tier=1), oracle_layer(case, tier=2))
    return _CASE_CACHE[key]


@pytest.mark.parametrize("name,small,tokens", LAYER_CASES)
@pytest.mark.parametrize("path", PATHS)
def test_layer_matches_checker(device, name, small, tokens, path):
    cfg, case, want, ideal = _case_and_reference(name, small, tokens)
    plan = make_plan(device, cfg, tokens, path)
    bank = ExpertBank.upload(device, case.w1, case.s1, case.w3, case.s3, case.w2, case.s2)
    hidden = device.resident_buffer_from(case.hidden)
    rw = device.resident_buffer_from(case.router_w)
    rbias = device.resident_buffer_from(case.router_bias) if case.router_bias is not None else None
    sbias = device.resident_buffer_from(case.select_bias) if case.select_bias is not None else None
    out = device.create_resident_buffer(tokens * cfg.hidden * 2)
    routes = device.create_resident_buffer(tokens * cfg.total_k * 4)
    logits = device.create_resident_buffer(want["logits"].nbytes)
    tele = device.create_resident_buffer(plan.telemetry_words() * 4)
    plan.layer(tokens, bank, hidden, out, router_weights=rw, router_bias=rbias, bias=sbias, routes_out=routes,
               logits=logits, telemetry=tele)
    np.testing.assert_array_equal(logits.read(np.uint32).reshape(want["logits"].shape), want["logits"])
    np.testing.assert_array_equal(routes.read(np.uint32).reshape(want["routes"].shape), want["routes"])
    got = out.read(np.uint16).reshape(tokens, cfg.hidden)
    m = assert_close(got, want["output"], f"{name} T{tokens} path{path}")
    assert plan.status() == 0
    hist = tele.read(np.uint32)[: cfg.total_experts]
    np.testing.assert_array_equal(hist, synthetic.expert_histogram(want["routes"], cfg.total_experts))
    report = plan.last_report()
    assert report["routes"] == tokens * cfg.total_k and report["kernel_launches"] > 0
    # the ideal tier (bf16 activations, no FP8 step) is reported, not gated: it measures the reference's
    # own activation quantisation, which this path reproduces
    print(f"\n{name} T{tokens} path{path}: vs same-operand reference {m}; vs unquantised-activation reference "
          f"{error_metrics(got, ideal['output'])}")
    plan.destroy()


@pytest.mark.parametrize("path", PATHS)
def test_layer_host_call_and_second_call_are_identical(device, path):
    cfg = synthetic.small_variant(synthetic.CONFIGS["gpt-oss-20b"], 256, 384, 16)
    tokens = 9
    case = synthetic.make_case(cfg, tokens, seed=2)
    plan = make_plan(device, cfg, 16, path)
    bank = ExpertBank.upload(device, case.w1, case.s1, case.w3, case.s3, case.w2, case.s2)
    rw = device.resident_buffer_from(case.router_w)
    rbias = device.resident_buffer_from(case.router_bias)
    out1 = np.zeros((tokens, cfg.hidden), dtype=np.uint16)
    out2 = np.zeros_like(out1)
    plan.layer_host(tokens, bank, case.hidden, out1, router_weights=rw, router_bias=rbias)
    plan.layer_host(tokens, bank, case.hidden, out2, router_weights=rw, router_bias=rbias)
    np.testing.assert_array_equal(out1, out2)
    want = oracle_layer(case, tier=1)
    assert_close(out1, want["output"])
    plan.destroy()


@pytest.mark.parametrize("path", PATHS)
def test_expert_ranges_partition_the_layer(device, path):
    """Expert-range ownership (expert_start/expert_count): each shard computes only the routes of
    the experts it owns; the shards' per-route rows tile the unpartitioned result exactly."""
    cfg = synthetic.small_variant(synthetic.CONFIGS["gpt-oss-120b"], 256, 256, 16)
    tokens = 40
    case = synthetic.make_case(cfg, tokens, seed=4)
    want = oracle_layer(case, tier=1)
    plan = make_plan(device, cfg, tokens, path)
    hidden = device.resident_buffer_from(case.hidden)
    rw = device.resident_buffer_from(case.router_w)
    rbias = device.resident_buffer_from(case.router_bias)
    out = device.create_resident_buffer(tokens * cfg.hidden * 2)
    full_bank = ExpertBank.upload(device, case.w1, case.s1, case.w3, case.s3, case.w2, case.s2)
    plan.layer(tokens, full_bank, hidden, out, router_weights=rw, router_bias=rbias)
    full = out.read(np.uint16).copy()
    assert_close(full, want["output"])
    acc = np.zeros((tokens, cfg.hidden), dtype=np.float64)
    for start in range(0, cfg.experts, 4):
        owned = list(range(start, start + 4))
        bank = ExpertBank.upload(device, case.w1, case.s1, case.w3, case.s3, case.w2, case.s2, present=owned)
        plan.layer(tokens, bank, hidden, out, router_weights=rw, router_bias=rbias, expert_start=start, expert_count=4)
        part = mo.bf16_to_f32(out.read(np.uint16)).reshape(tokens, cfg.hidden)
        # checker on the same ownership
        wpart = oracle_layer(case, tier=1, expert_start=start, expert_count=4)
        assert_close(out.read(np.uint16), wpart["output"], f"shard {start}")
        acc += part
        plan.status()
    ref = mo.bf16_to_f32(want["output"]).astype(np.float64)
    assert np.abs(acc - ref).max() <= 0.05 * np.abs(ref).max()
    plan.destroy()


@pytest.mark.parametrize("tokens", [24, 700, 1500])  # 700: several routes per thread of the one-block schedule; 1500: more than 16384 slots, the multi-block schedule
@pytest.mark.parametrize("path", PATHS)
def test_preselected_routes_form_reproduces_the_layer(device, path, tokens):
    """The owner's side of an expert-parallel exchange: the routes of a finished router arrive as rows
    of a top-1 plan (one hidden row and one route word per slot, unused slots marked 0xffffffff), the
    per-route rows come back instead of the combined output, and combining them reproduces the
    ordinary layer call bit for bit."""
    cfg = synthetic.small_variant(synthetic.CONFIGS["gpt-oss-120b"], 256, 384, 16)
    K, H = cfg.total_k, cfg.hidden
    case = synthetic.make_case(cfg, tokens, seed=8)
    plan = make_plan(device, cfg, tokens, path)
    bank = ExpertBank.upload(device, case.w1, case.s1, case.w3, case.s3, case.w2, case.s2)
    hidden = device.resident_buffer_from(case.hidden)
    rw = device.resident_buffer_from(case.router_w)
    rbias = device.resident_buffer_from(case.router_bias)
    out = device.create_resident_buffer(tokens * H * 2)
    routes_buf = device.create_resident_buffer(tokens * K * 4)
    plan.layer(tokens, bank, hidden, out, router_weights=rw, router_bias=rbias, routes_out=routes_buf)
    want = out.read(np.uint16).reshape(tokens, H).copy()
    routes = routes_buf.read(np.uint32).copy()

    # slots: every route twice over with gaps (slot 3*i holds route i), the rest unused
    slots = 3 * tokens * K + 5
    work_cfg = synthetic.MoeConfig(name="work", hidden=H, intermediate=cfg.intermediate, experts=cfg.total_experts, k=1,
                                   swiglu_limit=cfg.swiglu_limit, swiglu_alpha=cfg.swiglu_alpha,
                                   swiglu_up_offset=cfg.swiglu_up_offset, act_block=cfg.act_block)
    work = make_plan(device, work_cfg, slots, path)
    rows = np.zeros((slots, H), dtype=np.uint16)
    words = np.full(slots, 0xFFFFFFFF, dtype=np.uint32)
    where = 3 * np.arange(tokens * K)
    rows[where] = case.hidden[np.arange(tokens * K) // K]
    words[where] = routes
    rows_buf, words_buf = device.resident_buffer_from(rows), device.resident_buffer_from(words)
    per_slot = device.create_resident_buffer(slots * H * 2)
    for call in range(2):
        per_slot.fill(0x55)
        work.layer(slots, bank, rows_buf, None, routes_in=words_buf, expert_outputs=per_slot, expert_start=0,
                   expert_count=cfg.total_experts)
        got_rows = per_slot.read(np.uint16).reshape(slots, H)
        assert work.status() == 0
        expert_outputs = device.resident_buffer_from(np.ascontiguousarray(got_rows[where]))
        combined = device.create_resident_buffer(tokens * H * 2)
        plan.moe_reduce(tokens, expert_outputs, combined)
        np.testing.assert_array_equal(combined.read(np.uint16).reshape(tokens, H), want, err_msg=f"call {call}")
        unused = np.setdiff1d(np.arange(slots), where)
        assert not got_rows[unused].any(), "slots without a route must come back as zero rows"
    plan.destroy()
    work.destroy()


def test_bounded_wait_gives_up_and_the_plan_recovers(device):
    """A wait inside the tensor-core kernel that nothing will ever satisfy (CTA 0 leaves out one stage
    arrival) runs out after the plan's wait limit: the kernel returns, the status word says so, the
    context stays usable and the next ordinary call on the same plan is bit-identical to the one before.
    Nothing here faults, traps or hangs: the wait is bounded and simply expires."""
    cfg = synthetic.CONFIGS["tiny"]
    tokens = 64
    case = synthetic.make_case(cfg, tokens, seed=3)
    plan = make_plan(device, cfg, tokens, 2)
    bank = ExpertBank.upload(device, case.w1, case.s1, case.w3, case.s3, case.w2, case.s2)
    hidden = device.resident_buffer_from(case.hidden)
    rw = device.resident_buffer_from(case.router_w)
    out = device.create_resident_buffer(tokens * cfg.hidden * 2)
    plan.layer(tokens, bank, hidden, out, router_weights=rw)
    assert plan.status() == 0
    before = out.read(np.uint16).copy()
    plan.set_wait_limit(2_000_000)  # about a millisecond
    plan.debug_withhold_arrival(True)
    plan.layer(tokens, bank, hidden, out, router_weights=rw)
    device.synchronize(timeout_ns=20_000_000_000)
    assert plan.status() & 8, "NVMOE_STATUS_WAIT_EXPIRED must be raised when a bounded wait gives up"
    plan.debug_withhold_arrival(False)
    plan.set_wait_limit(0)
    for _ in range(2):
        plan.layer(tokens, bank, hidden, out, router_weights=rw)
        assert plan.status() == 0
        np.testing.assert_array_equal(out.read(np.uint16), before)
    plan.destroy()
