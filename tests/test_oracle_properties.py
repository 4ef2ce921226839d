"""Properties of the CPU checker that hold at any size, each against an independent numpy statement of
the shader rule it restates (no GPU, no reference checkout)."""
import numpy as np
import pytest

from oracle import moe_oracle as mo


def _bf16(x):
    return mo.bf16_to_f32(mo.f32_to_bf16(np.asarray(x, dtype=np.float32)))


def _logit_words(logits_f32):
    tokens, experts = logits_f32.shape
    half = np.zeros((tokens, 2 * ((experts + 1) // 2)), dtype=np.uint16)
    half[:, :experts] = mo.f32_to_bf16(logits_f32)
    return half.view(np.uint32)


@pytest.mark.parametrize("tokens,K,experts", [(1, 4, 32), (37, 4, 32), (64, 9, 257), (200, 2, 8)])
def test_histogram_compact_equals_the_quadratic_rank_of_the_shader(tokens, K, experts):
    """moe_route_compact_batch1.comp.template:87-105 ranks every route against every other one; the checker's
    counting sort must give the same permutation and control words."""
    rng = np.random.default_rng(tokens + experts)
    ids = np.stack([np.sort(rng.choice(experts, size=K, replace=False)) for _ in range(tokens)]).astype(np.uint32)
    routes = ((rng.integers(0, 1 << 16, size=(tokens, K), dtype=np.uint32) << 16) | ids).reshape(-1)
    I = 8
    frames = [np.zeros((tokens, K * I // 2 + K), dtype=np.uint32) for _ in range(2)]
    controls = [np.array([tokens, 0, 0, 0, 0, 0, 0], dtype=np.uint32) for _ in range(2)]
    mo.route_compact(routes, frames[0], controls[0], I, K, 3)
    mo.route_compact(routes, frames[1], controls[1], I, K, 3, quadratic=True)
    np.testing.assert_array_equal(frames[0], frames[1])
    np.testing.assert_array_equal(controls[0], controls[1])
    assert controls[0].tolist() == [tokens, 0, 0, tokens * K, K * 3, tokens, 1]
    order = frames[0][:, K * I // 2:].reshape(-1)
    assert sorted(order.tolist()) == list(range(tokens * K)), "the compact list is a permutation of the routes"
    keys = (routes[order] & 0xFFFF).astype(np.int64) * (tokens * K) + order
    assert np.all(np.diff(keys) > 0), "expert-major, source order inside an expert"
    assert not frames[0][:, : K * I // 2].any(), "the scheduler writes schedule words only"


@pytest.mark.parametrize("experts,k", [(8, 2), (32, 4), (128, 4)])
def test_softmax_over_selected_router_selects_the_top_k_and_normalises(experts, k):
    """moe_topk_bf16.comp.template:44-145: arg-max rounds on the raw logits with ties to the lower id, softmax
    over the k selected, routes ascending by id."""
    rng = np.random.default_rng(experts)
    tokens = 50
    logits = _bf16(rng.standard_normal((tokens, experts)) * 2.0)
    logits[3, :] = 0.5  # all tied: the k lowest ids win
    logits[4, 5] = logits[4, 1]
    p = mo.RouterParams(experts, k, kind=1, activation=1)
    telemetry = np.zeros(p.telemetry_words(), dtype=np.uint32)
    routes, bad = mo.route(p, _logit_words(logits), None, telemetry)
    assert bad == 0
    ids = (routes & 0xFFFF).astype(np.int64)
    weights = mo.bf16_to_f32((routes >> 16).astype(np.uint16)).astype(np.float64)
    assert np.all(np.diff(ids, axis=1) > 0)
    for t in range(tokens):
        want = np.lexsort((np.arange(experts), -logits[t].astype(np.float64)))[:k]  # value descending, id ascending
        assert sorted(want.tolist()) == ids[t].tolist(), f"token {t}"
        sel = logits[t, ids[t]].astype(np.float64)
        soft = np.exp(sel - sel.max())
        soft /= soft.sum()
        np.testing.assert_allclose(weights[t], soft, rtol=2.0 ** -8, atol=1e-6)
    assert ids[3].tolist() == list(range(k))
    assert telemetry[:experts].sum() == tokens * k
    assert telemetry[experts:].sum() == tokens * k * (k - 1) // 2
    np.testing.assert_array_equal(telemetry[:experts], np.bincount(ids.reshape(-1), minlength=experts))


def test_score_router_weights_come_from_the_activation_not_the_biased_score():
    """moe_router_score_topk_batch1_bf16.comp.template:127-187: selection on activation + bias, weight from the
    activation alone, normalised over the selected and scaled; the always-selected id is appended."""
    rng = np.random.default_rng(5)
    tokens, experts, k = 40, 64, 6
    logits = _bf16(rng.standard_normal((tokens, experts)))
    bias = (rng.standard_normal(experts) * 0.5).astype(np.float32)
    p = mo.RouterParams(experts, k, always_count=1, always_weight=1.0, kind=0, activation=0, normalize_selected=1,
                        bias_dtype=1, routed_scale=2.5)
    routes, bad = mo.route(p, _logit_words(logits), bias)
    assert bad == 0 and routes.shape == (tokens, k + 1)
    ids = (routes & 0xFFFF).astype(np.int64)
    weights = mo.bf16_to_f32((routes >> 16).astype(np.uint16)).astype(np.float64)
    assert np.all(ids[:, -1] == experts) and np.all(weights[:, -1] == 1.0)
    sig = 1.0 / (1.0 + np.exp(-logits.astype(np.float64)))
    for t in range(tokens):
        score = sig[t] + bias
        want = np.lexsort((np.arange(experts), -score))[:k]
        if np.min(np.diff(np.sort(score)[::-1][: k + 1])) < 1e-5:
            continue  # a near tie in f64 may fall the other way in f32
        assert sorted(want.tolist()) == ids[t, :k].tolist(), f"token {t}"
        act = sig[t, ids[t, :k]]
        np.testing.assert_allclose(weights[t, :k], act / act.sum() * 2.5, rtol=2.0 ** -7)


def test_combine_rounds_to_bf16_after_every_add_in_route_order():
    """moe_reduce_batch1_bf16.comp.template:29-55."""
    rng = np.random.default_rng(9)
    tokens, K, hidden = 17, 4, 96
    rows = mo.f32_to_bf16(rng.standard_normal((tokens, K, hidden)).astype(np.float32) * 3.0)
    got = mo.reduce(rows, tokens, K, hidden, routed_scale=0.5)
    acc = np.zeros((tokens, hidden), dtype=np.float32)
    for r in range(K):
        acc = _bf16(acc + mo.bf16_to_f32(rows[:, r, :]))
    np.testing.assert_array_equal(got, mo.f32_to_bf16(acc * np.float32(0.5)))
    # the order matters: a different order gives different bits somewhere, which is why it is pinned
    other = np.zeros((tokens, hidden), dtype=np.float32)
    for r in reversed(range(K)):
        other = _bf16(other + mo.bf16_to_f32(rows[:, r, :]))
    assert np.any(mo.f32_to_bf16(other * np.float32(0.5)) != got)


@pytest.mark.parametrize("block", [32, 128])
def test_activation_quantisation_is_exact_for_representable_values_and_bounded_otherwise(block):
    """…gate_up_batch1_mxfp4.comp.template:357-383: one power-of-two scale per block, E4M3 codes."""
    rng = np.random.default_rng(block)
    rows, cols = 9, 4 * block
    x = mo.f32_to_bf16((rng.standard_normal((rows, cols)) * np.exp(rng.uniform(-6, 6, (rows, 1)))).astype(np.float32))
    x[0, :block] = 0  # an all-zero block takes the floor scale
    q, scales = mo.quantize_fp8(x, block)
    xf = mo.bf16_to_f32(x).reshape(rows, cols // block, block).astype(np.float64)
    peak = np.maximum(np.abs(xf).max(axis=2), 1e-4)
    assert np.all(np.log2(scales) == np.round(np.log2(scales))), "scales are powers of two"
    assert np.all(scales.astype(np.float64) * 448.0 >= peak) and np.all(scales.astype(np.float64) * 224.0 < peak * (1 + 1e-6))
    table = np.array([mo.lib().oracle_e4m3_value(b) for b in range(256)], dtype=np.float64)
    back = table[q].reshape(rows, cols // block, block) * scales[:, :, None]
    # E4M3 keeps 3 mantissa bits: relative error at most 2^-4 for normal codes, absolute 2^-10 * scale below them
    err = np.abs(back - xf)
    assert np.all(err <= np.maximum(np.abs(xf) * 2.0 ** -4, scales[:, :, None] * 2.0 ** -10) * (1 + 1e-9))
    assert not q[0, :block].any()
