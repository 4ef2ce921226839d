"""The CPU checker against the reference's own golden vectors and known answers.

Fixtures in tests/golden/reference_vectors.json were produced by tests/golden/make_golden.py,
which imports the Python half of the reference; the Rust/Vulkan known answers in it were
transcribed by reading the reference's GPU-only tests (file:line in that script).
"""
import json
import math
from fractions import Fraction
from pathlib import Path

import numpy as np
import pytest

from oracle import moe_oracle as mo

GOLDEN = json.loads((Path(__file__).parent / "golden" / "reference_vectors.json").read_text())
L = mo.lib()


def test_e2m1_tables_match_reference_tables():
    t = GOLDEN["tables"]
    for nibble in range(16):
        assert L.oracle_e2m1_to_e4m3(nibble) == t["e4m3_bits"][nibble]
        assert L.oracle_e2m1_value(nibble) * 2 == t["sint8_codes"][nibble]
    # tests/test_quantized_transforms.py:22-27 and :38-42 (low nibble first)
    packed = t["expand_e4m3"]["input"]
    out = []
    for byte in packed:
        out += [L.oracle_e2m1_to_e4m3(byte & 0xF), L.oracle_e2m1_to_e4m3(byte >> 4)]
    assert out == t["expand_e4m3"]["output"]
    out = []
    for byte in t["expand_sint8"]["input"]:
        out += [int(L.oracle_e2m1_value(byte & 0xF) * 2) & 0xFF, int(L.oracle_e2m1_value(byte >> 4) * 2) & 0xFF]
    assert out == t["expand_sint8"]["output"]


def test_every_nibble_scale_pair_is_exact():
    t = GOLDEN["tables"]
    for scale in range(0xFF):
        s = Fraction(*t["e8m0"][str(scale)])
        assert Fraction(float(L.oracle_e8m0_value(scale))) == s
        for nibble in range(16):
            want = Fraction(*t["mxfp4_value"][f"{nibble}:{scale}"])
            got = Fraction(float(L.oracle_e2m1_value(nibble))) * Fraction(float(L.oracle_e8m0_value(scale)))
            assert got == want


def test_e4m3_decode_matches_reference_for_every_byte():
    for bits in range(256):
        want = Fraction(*GOLDEN["tables"]["e4m3_value"][str(bits)])
        assert Fraction(float(L.oracle_e4m3_value(bits))) == want


def test_numpy_decoder_of_the_reference_agrees():
    g = GOLDEN["numpy_decoder"]
    packed = np.array(g["packed"], dtype=np.uint8).reshape(g["rows"], g["cols"] // 2)
    scales = np.array(g["scales"], dtype=np.uint8).reshape(g["rows"], g["cols"] // 32)
    want = np.array(g["decoded_f32_bits"], dtype=np.uint32).view(np.float32).reshape(g["rows"], g["cols"])
    got = mo.dequant_mxfp4(packed, scales)
    # the reference decoder flushes nothing: compare bit patterns (signed zeros included)
    np.testing.assert_array_equal(got.view(np.uint32), want.view(np.uint32))


def test_f32_to_e4m3_round_trips_and_rounds_to_nearest_even():
    torch = pytest.importorskip("torch")
    for bits in range(256):
        if (bits & 0x7F) == 0x7F:
            continue
        assert L.oracle_f32_to_e4m3(L.oracle_e4m3_value(bits)) == bits or (bits & 0x7F) == 0  # -0 ok below
    assert L.oracle_f32_to_e4m3(-0.0) == 0x80
    rng = np.random.default_rng(7)
    x = np.concatenate([
        rng.uniform(-448, 448, 20000), rng.normal(0, 1, 20000), rng.normal(0, 0.01, 20000),
        np.array([0.0, 448.0, -448.0, 2.0 ** -9, 2.0 ** -10, 3 * 2.0 ** -10, 2.0 ** -6, 0.0175, 17.0, 18.0, 19.0]),
    ]).astype(np.float32)
    want = torch.from_numpy(x).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    got = np.array([L.oracle_f32_to_e4m3(float(v)) for v in x], dtype=np.uint8)
    np.testing.assert_array_equal(got, want)


def test_bf16_rounding_matches_torch():
    torch = pytest.importorskip("torch")
    rng = np.random.default_rng(3)
    x = rng.normal(0, 10, 50000).astype(np.float32)
    want = torch.from_numpy(x).to(torch.bfloat16).view(torch.uint16).numpy()
    np.testing.assert_array_equal(mo.f32_to_bf16(x), want)
    assert [L.oracle_f32_to_bf16(float(v)) for v in x[:100]] == list(want[:100])


def _ulp_diff(a, b):
    a = np.asarray(a, dtype=np.float32)
    b = np.asarray(b, dtype=np.float32)
    return np.abs(a.view(np.int32).astype(np.int64) - b.view(np.int32).astype(np.int64))


def test_pinned_transcendentals_are_accurate():
    xs = np.linspace(-87, 88, 20001).astype(np.float32)
    got = np.array([L.oracle_expf(float(v)) for v in xs], dtype=np.float32)
    assert _ulp_diff(got, np.exp(xs.astype(np.float64)).astype(np.float32)).max() <= 2
    xs = np.concatenate([np.linspace(1e-6, 4, 20001), np.logspace(-30, 30, 2001)]).astype(np.float32)
    got = np.array([L.oracle_logf(float(v)) for v in xs], dtype=np.float32)
    want = np.log(xs.astype(np.float64)).astype(np.float32)
    assert np.all(np.abs(got - want) <= 4e-7 * np.maximum(1.0, np.abs(want)))
    xs = np.linspace(-12, 12, 20001).astype(np.float32)
    got = np.array([L.oracle_tanhf(float(v)) for v in xs], dtype=np.float32)
    assert np.abs(got - np.tanh(xs.astype(np.float64))).max() <= 3e-7
    assert L.oracle_expf(-200.0) == 0.0 and math.isinf(L.oracle_expf(100.0))


def test_activation_scale_is_smallest_power_of_two_not_below_max_over_448():
    for m in [0.0, 1e-5, 1e-4, 0.3, 1.0, 447.9, 448.0, 448.1, 896.0, 1e6]:
        s = L.oracle_rounded_fp8_scale(m)
        ratio = max(m, 1e-4) / 448.0
        assert math.log2(s) == int(math.log2(s))
        assert s >= np.float32(ratio) and s / 2 < np.float32(ratio) * (1 + 1e-7)


# ---- constant-fill known answers of the reference's Vulkan conformance tests -------------------

def _fill_case(width, experts, fills, k):
    w = {e: np.full((width, width // 2), fills[e], dtype=np.uint8) for e in fills}
    s = {e: np.full((width, width // 32), 120, dtype=np.uint8) for e in fills}
    return w, s


def test_constant_fill_gate_up_down_known_answers():
    ka = GOLDEN["rust_known_answers"]["constant_fill"]
    W = ka["width"]
    p = mo.ExpertParams(W, W, 1, 1, tile_rows=32, swiglu_limit=ka["swiglu_limit"], act_block=128, tier=0)
    hidden = mo.f32_to_bf16(np.ones((1, W), dtype=np.float32))
    routes = np.array([[int(mo.f32_to_bf16(np.array([1.0]))[0]) << 16]], dtype=np.uint32)
    wt = np.full((W, W // 2), ka["weight_fill"], dtype=np.uint8)
    sc = np.full((W, W // 32), ka["scale_fill"], dtype=np.uint8)
    addr = mo.address_table([wt, sc, wt, sc])
    slots = np.array([0, 1, 2, 3], dtype=np.uint32)
    expected = int(mo.f32_to_bf16(np.array([1.0 / (1.0 + np.exp(np.float32(-1.0)))], dtype=np.float32))[0])
    for tier in (0, 1, 2):
        p.tier = tier
        inter = np.zeros((1, p.frame_words), dtype=np.uint32)
        control = np.array([1, 0, 0, 0, 4, 1, 1], dtype=np.uint32)
        mo.gate_up(p, hidden, routes, inter, addr, slots, control)
        data = inter[0, : p.data_words].view(np.uint16)
        assert np.all(data == expected), tier
    # prequantised twin: bytes 0x38 (=1.0) with scale 1.0 (mxfp4_tests.rs:134-162)
    p.tier = 0
    inter = np.zeros((1, p.frame_words), dtype=np.uint32)
    mo.gate_up_prequant(p, np.full((1, W), 0x38, dtype=np.uint8), np.ones((1, 1), dtype=np.float32),
                        routes, inter, addr, slots, np.array([1, 0, 0, 0, 4, 1, 1], dtype=np.uint32))
    assert np.all(inter[0, : p.data_words].view(np.uint16) == expected)
    # down: intermediates of 1.0 -> outputs of 1.0, then every E2M1 code (mxfp4_tests.rs:164-215)
    one = int(mo.f32_to_bf16(np.array([1.0], dtype=np.float32))[0])
    inter = np.zeros((1, p.frame_words), dtype=np.uint32)
    inter[0, : p.data_words] = one | (one << 16)
    daddr = mo.address_table([wt, sc])
    dslots = np.array([0, 1], dtype=np.uint32)
    out = np.zeros((1, 1, W), dtype=np.uint16)
    mo.down(p, inter, routes, out, daddr, dslots, np.array([1, 0, 0, 0, 2, 1, 1], dtype=np.uint32))
    assert np.all(out == one)
    for nibble, value in enumerate(ka["e2m1_values"]):
        wt[:] = nibble | (nibble << 4)
        out[:] = 0
        mo.down(p, inter, routes, out, daddr, dslots, np.array([1, 0, 0, 0, 2, 1, 1], dtype=np.uint32))
        assert np.all(mo.bf16_to_f32(out) == np.float32(value)), nibble


def test_fail_closed_on_invalid_metadata():
    W = 128
    p = mo.ExpertParams(W, W, 1, 1, swiglu_limit=10.0, tier=0)
    routes = np.array([[0x3F80 << 16]], dtype=np.uint32)
    wt = np.full((W, W // 2), 0x22, dtype=np.uint8)
    sc = np.full((W, W // 32), 120, dtype=np.uint8)
    addr = mo.address_table([wt, sc, wt, sc])
    slots = np.array([0, 1, 2, 3], dtype=np.uint32)
    q = np.full((1, W), 0x38, dtype=np.uint8)
    one = np.ones((1, 1), dtype=np.float32)
    control = np.array([1, 0, 0, 0, 0, 0, 0], dtype=np.uint32)
    inter = np.zeros((1, p.frame_words), dtype=np.uint32)
    inter[0, p.data_words] = 0xFFFFFFFF  # out-of-range compact route
    mo.gate_up_prequant(p, q, one, routes, inter, addr, slots, control)
    assert np.all(inter[0, : p.data_words] == 0)
    inter[0, p.data_words] = 0
    mo.gate_up_prequant(p, q, one, routes, inter, np.zeros_like(addr), slots, control)  # unpublished records
    assert np.all(inter[0, : p.data_words] == 0)
    for bad_word, value in ((4, 0), (6, 0), (6, 2), (2, 16), (0, addr[0] | 1), (7, 1)):
        broken = addr.copy()
        broken[bad_word] = value
        if bad_word == 4:
            broken[5] = 0
        inter[:] = 0
        mo.gate_up_prequant(p, q, one, routes, inter, broken, slots, control)
        assert np.all(inter[0, : p.data_words] == 0), (bad_word, value)
    bad_slots = slots.copy()
    bad_slots[2] = 0xFFFFFFFF
    mo.gate_up_prequant(p, q, one, routes, inter, addr, bad_slots, control)
    assert np.all(inter[0, : p.data_words] == 0)
    mo.gate_up_prequant(p, q, one, routes, inter, addr, slots, control)
    assert np.all(inter[0, : p.data_words] != 0)


def test_route_native_matches_canonical_and_control_words():
    ka = GOLDEN["rust_known_answers"]["route_native"]
    H, I, E, K = ka["hidden"], ka["intermediate"], ka["experts"], ka["k"]
    p = mo.ExpertParams(H, I, E, K, tile_rows=32, swiglu_limit=10.0, tier=0)
    routes = np.array([[e | (int(mo.f32_to_bf16(np.array([w], dtype=np.float32))[0]) << 16) for e, w in ka["routes"]]],
                      dtype=np.uint32)
    q = np.full((1, H), 0x38, dtype=np.uint8)
    one = np.ones((1, 1), dtype=np.float32)
    keep = []
    gres, gslots = [], np.full(E * 4, mo.UNBOUND_SLOT, dtype=np.uint32)
    dres, dslots = [], np.full(E * 2, mo.UNBOUND_SLOT, dtype=np.uint32)
    for e in ka["bound_experts"]:
        fill = ka["fills"][str(e)]
        for j in range(4):
            arr = np.full((I, H // 2) if j % 2 == 0 else (I, H // 32), fill if j % 2 == 0 else ka["scale_fill"], dtype=np.uint8)
            gslots[e * 4 + j] = len(gres)
            gres.append(arr)
        for j in range(2):
            arr = np.full((H, I // 2) if j == 0 else (H, I // 32), fill if j == 0 else ka["scale_fill"], dtype=np.uint8)
            dslots[e * 2 + j] = len(dres)
            dres.append(arr)
    gaddr, daddr = mo.address_table(gres), mo.address_table(dres)

    def run(route_native):
        inter = np.zeros((1, p.frame_words), dtype=np.uint32)
        inter[0, p.data_words:] = np.arange(K)  # reset_intermediates of the reference test
        if route_native:
            gc = np.array(ka["control_in"], dtype=np.uint32)
            dc = np.array(ka["control_in"], dtype=np.uint32)
            mo.route_compact(routes, inter, gc, I, K, -(-I // 32))
            mo.route_count(routes, dc, K, -(-H // 64))
            assert gc.tolist() == ka["gate_control_out"]
            assert dc.tolist() == ka["down_control_out"]
        else:
            gc = np.array(ka["canonical_control"]["gate"], dtype=np.uint32)
            dc = np.array(ka["canonical_control"]["down"], dtype=np.uint32)
        mo.gate_up_prequant(p, q, one, routes, inter, gaddr, gslots, gc)
        out = np.zeros((1, K, H), dtype=np.uint16)
        mo.down(p, inter, routes, out, daddr, dslots, dc)
        return out

    canonical, native = run(False), run(True)
    np.testing.assert_array_equal(canonical, native)
    assert canonical.any()


def test_tp_partial_reduction_equals_canonical_scaling():
    # one participant: f32 partial x packed bf16 route weight == canonical bf16 output
    # (mxfp4_route_native_tests.rs:252-434)
    ka = GOLDEN["rust_known_answers"]["tp_reduction"]
    H = I = 128
    K = 2
    p = mo.ExpertParams(H, I, 4, K, tier=0)
    inter = np.zeros((1, p.frame_words), dtype=np.uint32)
    inter[0, p.data_words:] = np.arange(K)
    inter[0, : p.data_words] = (ka["intermediate_word_base"] + np.arange(p.data_words)).astype(np.uint32)
    routes = np.array([[3 | (0x3F40 << 16), 1 | (0x3E80 << 16)]], dtype=np.uint32)
    res, slots = [], np.full(8, mo.UNBOUND_SLOT, dtype=np.uint32)
    for e, fill in ((1, 0x22), (3, 0x44)):
        slots[e * 2], slots[e * 2 + 1] = len(res), len(res) + 1
        res += [np.full((H, I // 2), fill, dtype=np.uint8), np.full((H, I // 32), 120, dtype=np.uint8)]
    addr = mo.address_table(res)
    control = np.array([1, 0, 0, 0, K * 2, 1, 1], dtype=np.uint32)
    canonical = np.zeros((1, K, H), dtype=np.uint16)
    mo.down(p, inter, routes, canonical, addr, slots, control)
    # unscaled f32 partials: rerun with weight 1.0 routes in the f64 tier is not the same thing;
    # rebuild them from the dequantised matrices and the quantised intermediates instead
    partials = np.zeros((K, H), dtype=np.float32)
    for r in range(K):
        expert = int(routes[0, r] & 0xFFFF)
        unit = routes.copy()
        unit[0, r] = expert | (0x3F80 << 16)
        o = np.zeros((1, K, H), dtype=np.uint16)
        # a route weight of 1.0 leaves value * 1.0, but rounds to bf16: take the f32 by hand
        x = mo.bf16_to_f32(inter[0, : p.data_words].view(np.uint16)[r * I:(r + 1) * I].copy())
        qx, sx = mo.quantize_fp8(mo.f32_to_bf16(x)[None, :], 128)
        deq = np.array([L.oracle_e4m3_value(int(b)) for b in qx[0]], dtype=np.float64) * np.repeat(sx[0].astype(np.float64), 128)
        wmat = mo.dequant_mxfp4(res[slots[expert * 2]], res[slots[expert * 2 + 1]]).astype(np.float64)
        partials[r] = (wmat @ deq).astype(np.float32)
    push = ka["reduction_push"]
    out_words = mo.sum_f32_scale_packed_bf16(partials.reshape(-1), routes.reshape(-1), push[0], push[1], push[2], push[3], push[4])
    np.testing.assert_array_equal(out_words.view(np.uint16), canonical.reshape(-1))
