"""GPU parity of the integer-exact part of the path: router projection, the three router forms,
route scheduling and activation quantisation — all bit-exact against the CPU checker, through the
C ABI."""
import zlib

import numpy as np
import pytest

from nerve_b200 import synthetic
from nerve_b200.backend import CudaComputeDevice, MoePlan, geometry_from_config
from oracle import moe_oracle as mo
from tests.helpers import router_params

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def device():
    dev = CudaComputeDevice(0)
    yield dev
    dev.close()


def _cfg(experts, k, **kw):
    base = dict(name="t", hidden=256, intermediate=256, experts=experts, k=k, act_block=128)
    base.update(kw)
    return synthetic.MoeConfig(**base)


@pytest.mark.parametrize("tokens,hidden,experts,bias", [(1, 2880, 32, True), (7, 256, 8, False), (64, 2880, 32, True),
                                                         (33, 7168, 257, False), (300, 512, 130, True)])
def test_router_projection_is_bit_exact(device, tokens, hidden, experts, bias):
    rng = np.random.default_rng(tokens * 1000 + experts)
    x = synthetic.f32_to_bf16(rng.standard_normal((tokens, hidden), dtype=np.float32))
    w = synthetic.f32_to_bf16(0.02 * rng.standard_normal((experts, hidden), dtype=np.float32))
    b = synthetic.f32_to_bf16(0.1 * rng.standard_normal(experts).astype(np.float32)) if bias else None
    want = mo.linear_bf16(x, w, b)
    plan = MoePlan(device, geometry_from_config(_cfg(experts, 1, hidden=hidden, intermediate=128, act_block=32), tokens))
    xb, wb = device.resident_buffer_from(x), device.resident_buffer_from(w)
    bb = device.resident_buffer_from(b) if bias else None
    lb = device.create_resident_buffer(want.nbytes)
    plan.linear(tokens, xb, lb, wb, bb)
    got = lb.read(np.uint32).reshape(want.shape)
    np.testing.assert_array_equal(got, want)
    plan.destroy()


ROUTER_CASES = [
    # score_topk: sigmoid / softmax-over-all / sqrt-softplus, with and without bias, normalise, always-selected
    dict(experts=8, k=2, router_kind=0, activation=1, normalize_selected=1),
    dict(experts=256, k=8, router_kind=0, activation=0, normalize_selected=1, routed_scale=2.5, bias_dtype=1,
         always_count=1, always_weight=1.0),
    dict(experts=256, k=8, router_kind=0, activation=0, normalize_selected=1, routed_scale=2.5, bias_dtype=1,
         always_count=1, n_group=8, topk_group=4),
    dict(experts=64, k=6, router_kind=0, activation=2, normalize_selected=0, routed_scale=1.5, bias_dtype=2),
    dict(experts=160, k=6, router_kind=0, activation=1, normalize_selected=0, always_count=2, always_weight=0.5),
    dict(experts=1000, k=10, router_kind=0, activation=1, normalize_selected=1),
    # softmax over the selected k
    dict(experts=32, k=4, router_kind=1),
    dict(experts=128, k=4, router_kind=1),
    dict(experts=7, k=7, router_kind=1),
    # routed top-k: soft-cap, sigmoid or softmax, selection bias, normalise flag
    dict(experts=128, k=8, router_kind=2, activation=0, normalize_selected=1, bias_dtype=1),
    dict(experts=128, k=8, router_kind=2, activation=1, normalize_selected=0, logit_softcap=30.0),
    dict(experts=60, k=4, router_kind=2, activation=1, normalize_selected=1, bias_dtype=2, logit_softcap=5.0),
    dict(experts=60, k=4, router_kind=2, activation=0, normalize_selected=0),
]


@pytest.mark.parametrize("case", ROUTER_CASES, ids=lambda c: "-".join(f"{k}{v}" for k, v in c.items()))
@pytest.mark.parametrize("tokens", [1, 97])
def test_routes_and_telemetry_are_bit_exact(device, case, tokens):
    cfg = _cfg(**case)
    rp = router_params(cfg)
    rng = np.random.default_rng(zlib.crc32(str(sorted(case.items())).encode()) + tokens)
    # coarse logits give plenty of exact ties, which must go to the lower expert index
    logits_f = np.round(rng.standard_normal((tokens, cfg.experts)) * 4) / 4
    lw = np.zeros((tokens, (cfg.experts + 1) // 2 * 2), dtype=np.uint16)
    lw[:, : cfg.experts] = synthetic.f32_to_bf16(logits_f.astype(np.float32))
    logit_words = lw.view(np.uint32)
    bias = None
    if cfg.bias_dtype == 1:
        bias = (np.round(rng.standard_normal(cfg.experts) * 8) / 64).astype(np.float32)
    elif cfg.bias_dtype == 2:
        bias = synthetic.f32_to_bf16((0.05 * rng.standard_normal(cfg.experts)).astype(np.float32))
    tele_want = np.zeros(rp.telemetry_words(), dtype=np.uint32)
    want, bad = mo.route(rp, logit_words, bias, tele_want)
    assert bad == 0

    plan = MoePlan(device, geometry_from_config(cfg, tokens))
    lb = device.resident_buffer_from(logit_words)
    bb = device.resident_buffer_from(bias) if bias is not None else None
    rb = device.create_resident_buffer(want.nbytes)
    tb = device.create_resident_buffer(tele_want.nbytes)
    plan.moe_route(tokens, lb, rb, bb, tb)
    got = rb.read(np.uint32).reshape(want.shape)
    np.testing.assert_array_equal(got & 0xFFFF, want & 0xFFFF, err_msg="expert ids")
    np.testing.assert_array_equal(got >> 16, want >> 16, err_msg="bf16 route weights")
    np.testing.assert_array_equal(tb.read(np.uint32), tele_want)
    ids = (got & 0xFFFF).astype(np.int64)
    assert np.all(np.diff(ids, axis=1) > 0), "routes must ascend by expert id within a token"
    assert plan.status() == 0
    plan.destroy()


def test_router_fails_closed_on_nan_logits(device):
    cfg = _cfg(8, 2, router_kind=1)
    plan = MoePlan(device, geometry_from_config(cfg, 2))
    lw = np.zeros((2, 8), dtype=np.uint16)
    lw[0, :] = 0x7FC0  # NaN
    lw[1, :] = synthetic.f32_to_bf16(np.arange(8, dtype=np.float32))
    lb = device.resident_buffer_from(lw.view(np.uint32))
    rb = device.create_resident_buffer(2 * 2 * 4)
    plan.moe_route(2, lb, rb)
    got = rb.read(np.uint32).reshape(2, 2)
    assert np.all(got[0] == 0)
    assert (got[1] & 0xFFFF).tolist() == [6, 7]
    assert plan.status() & 1
    plan.destroy()


def _random_routes(rng, tokens, K, experts):
    ids = np.stack([np.sort(rng.choice(experts, K, replace=False)) for _ in range(tokens)]).astype(np.uint32)
    w = synthetic.f32_to_bf16(rng.random((tokens, K), dtype=np.float32)).astype(np.uint32)
    return (w << 16) | ids


@pytest.mark.parametrize("tokens,K,experts,I", [(1, 4, 32, 64), (64, 4, 32, 2880), (1000, 4, 32, 64), (2500, 9, 257, 32),
                                                (4096, 4, 32, 32),
                                                (8192, 4, 128, 32),     # 32 768 routes: the gpt-oss-120b batch
                                                (16384, 9, 257, 32)])   # 147 456 routes: the DeepSeek-V3 batch
def test_compact_rank_mode_matches_reference_ranking(device, tokens, K, experts, I):
    rng = np.random.default_rng(tokens + K)
    cfg = _cfg(experts, K, hidden=64, intermediate=I, act_block=32)
    plan = MoePlan(device, geometry_from_config(cfg, tokens))
    routes = _random_routes(rng, tokens, K, experts)
    frame = plan.frame_words
    want_inter = np.zeros((tokens, frame), dtype=np.uint32)
    want_control = np.array([tokens, 0, 0, 0, 0, 0, 0], dtype=np.uint32)
    tiles = -(-I // 32)
    mo.route_compact(routes, want_inter, want_control, I, K, tiles)
    if tokens * K <= 4000:
        check = np.zeros_like(want_inter)
        cc = np.array([tokens, 0, 0, 0, 0, 0, 0], dtype=np.uint32)
        mo.route_compact(routes, check, cc, I, K, tiles, quadratic=True)  # the shader's own quadratic ranking
        np.testing.assert_array_equal(check, want_inter)
    rb = device.resident_buffer_from(routes)
    ib = device.create_resident_buffer(want_inter.nbytes)
    cb = device.resident_buffer_from(np.array([tokens, 0, 0, 0, 0, 0, 0], dtype=np.uint32))
    plan.moe_route_compact(tokens, rb, ib, cb)
    got = ib.read(np.uint32).reshape(tokens, frame)
    np.testing.assert_array_equal(got[:, plan.data_words:], want_inter[:, plan.data_words:])
    assert not got[:, : plan.data_words].any(), "the scheduler must not touch the data words"
    np.testing.assert_array_equal(cb.read(np.uint32), want_control)
    # down-stage counter
    dc = device.resident_buffer_from(np.array([tokens, 0, 0, 0, 0, 0, 0], dtype=np.uint32))
    plan.moe_route_count(tokens, rb, dc)
    wc = np.array([tokens, 0, 0, 0, 0, 0, 0], dtype=np.uint32)
    mo.route_count(routes, wc, K, -(-64 // 64))
    np.testing.assert_array_equal(dc.read(np.uint32), wc)
    plan.destroy()


@pytest.mark.parametrize("tokens,K,experts,start,count,with_slots", [(1, 2, 4, 0, 4, True), (64, 4, 32, 8, 8, False),
                                                                      (3000, 4, 32, 16, 16, True), (700, 9, 257, 128, 129, True)])
def test_compact_partitioned_mode_filters_owned_routes_in_source_order(device, tokens, K, experts, start, count, with_slots):
    rng = np.random.default_rng(tokens * 7 + K)
    I = 64
    cfg = _cfg(experts, K, hidden=64, intermediate=I, act_block=32)
    plan = MoePlan(device, geometry_from_config(cfg, tokens))
    routes = _random_routes(rng, tokens, K, experts)
    gslots = dslots = None
    if with_slots:
        gslots = np.arange(experts * 4, dtype=np.uint32)
        dslots = np.arange(experts * 2, dtype=np.uint32)
        for e in rng.choice(experts, max(experts // 5, 1), replace=False):
            gslots[e * 4: e * 4 + 4] = 0xFFFFFFFF
            dslots[e * 2: e * 2 + 2] = 0xFFFFFFFF
    want_inter = np.zeros((tokens, plan.frame_words), dtype=np.uint32)
    wc = np.array([tokens, start, count, 0, 0, 0, 0], dtype=np.uint32)
    mo.route_compact(routes, want_inter, wc, I, K, 2, slots=gslots)
    rb = device.resident_buffer_from(routes)
    ib = device.create_resident_buffer(want_inter.nbytes)
    cb = device.resident_buffer_from(np.array([tokens, start, count, 0, 0, 0, 0], dtype=np.uint32))
    sb = device.resident_buffer_from(gslots) if with_slots else None
    plan.moe_route_compact(tokens, rb, ib, cb, sb)
    got_control = cb.read(np.uint32)
    np.testing.assert_array_equal(got_control, wc)
    owned = int(wc[3])
    got = ib.read(np.uint32).reshape(tokens, plan.frame_words)[:, plan.data_words:].reshape(-1)[:owned]
    want = want_inter[:, plan.data_words:].reshape(-1)[:owned]
    np.testing.assert_array_equal(got, want)
    dc = device.resident_buffer_from(np.array([tokens, start, count, 0, 0, 0, 0], dtype=np.uint32))
    db = device.resident_buffer_from(dslots) if with_slots else None
    plan.moe_route_count(tokens, rb, dc, db)
    wdc = np.array([tokens, start, count, 0, 0, 0, 0], dtype=np.uint32)
    mo.route_count(routes, wdc, K, 1, slots=dslots)
    np.testing.assert_array_equal(dc.read(np.uint32), wdc)
    plan.destroy()


@pytest.mark.parametrize("rows,cols,block", [(1, 128, 128), (5, 2880, 32), (64, 7168, 128), (300, 256, 64)])
def test_activation_quantisation_is_bit_exact(device, rows, cols, block):
    rng = np.random.default_rng(rows + cols)
    x = rng.standard_normal((rows, cols), dtype=np.float32) * rng.choice([1e-3, 1.0, 50.0], (rows, 1)).astype(np.float32)
    x[0, :block] = 0.0  # an all-zero block takes the 1e-4 floor
    xb16 = synthetic.f32_to_bf16(x)
    wq, ws = mo.quantize_fp8(xb16, block)
    cfg = _cfg(4, 1, hidden=cols, intermediate=cols, act_block=block)
    plan = MoePlan(device, geometry_from_config(cfg, rows))
    ib = device.resident_buffer_from(xb16)
    qb = device.create_resident_buffer(wq.nbytes)
    sb = device.create_resident_buffer(ws.nbytes)
    plan.quantize_fp8_e4m3(rows, cols, ib, qb, sb)
    np.testing.assert_array_equal(qb.read(np.uint8).reshape(wq.shape), wq)
    np.testing.assert_array_equal(sb.read(np.float32).reshape(ws.shape), ws)
    plan.destroy()
