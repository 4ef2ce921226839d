"""GPU parity of the nodes around the MoE chain (ffn_norm, the dense shared expert, the residual add), of
the token-id table routing, and of a whole feed-forward block run node by node from the compiler's own
node list.  Elementwise and integer results are compared bit for bit with the CPU checker; the dense
linears within the tolerance of the expert projections they share kernels with."""
import copy
import json
from pathlib import Path

import numpy as np
import pytest

from nerve_b200 import synthetic
from nerve_b200.backend import CudaComputeDevice, ExpertBank, MoePlan, geometry_from_config
from nerve_b200.node_chain import plan_from_nodes
from oracle import moe_oracle as mo
from tests.helpers import assert_close, oracle_layer

pytestmark = pytest.mark.gpu
GOLDEN = json.loads((Path(__file__).parent / "golden" / "reference_vectors.json").read_text())["node_chain"]


@pytest.fixture(scope="module")
def device():
    dev = CudaComputeDevice(0)
    yield dev
    dev.close()


def bf16(x):
    return synthetic.f32_to_bf16(np.asarray(x, dtype=np.float32))


def small_plan(device, hidden=256, intermediate=384, tokens=64, act_block=32, path=0, **kw):
    cfg = synthetic.MoeConfig("ffn", hidden, intermediate, 8, 2, act_block=act_block, **kw)
    plan = MoePlan(device, geometry_from_config(cfg, tokens))
    if path:
        plan.set_expert_path(path)
    return cfg, plan


@pytest.mark.parametrize("rows,hidden,eps,offset", [(1, 128, 1e-6, 0.0), (37, 2880, 1e-5, 0.0), (64, 7168, 1e-6, 1.0), (5, 130, 1e-6, 0.0)])
def test_rms_norm_is_bit_exact(device, rows, hidden, eps, offset):
    rng = np.random.default_rng(rows + hidden)
    x = bf16(rng.standard_normal((rows, hidden)) * rng.choice([1e-2, 1.0, 30.0], (rows, 1)))
    w = bf16(1.0 + 0.1 * rng.standard_normal(hidden))
    _, plan = small_plan(device)
    xb, wb = device.resident_buffer_from(x), device.resident_buffer_from(w)
    ob = device.create_resident_buffer(x.nbytes)
    plan.rms_norm(rows, hidden, xb, ob, wb, eps, offset)
    np.testing.assert_array_equal(ob.read(np.uint16).reshape(x.shape), mo.rms_norm(x, w, eps, offset))
    plan.destroy()


@pytest.mark.parametrize("rows,count,limit", [(1, 128, 0.0), (33, 2880, 7.0), (64, 2048, 0.0), (3, 6, 10.0)])
def test_silu_multiply_both_forms_and_residual_add_are_bit_exact(device, rows, count, limit):
    rng = np.random.default_rng(rows * 7 + count)
    g = bf16(rng.standard_normal((rows, count)) * 6.0)
    u = bf16(rng.standard_normal((rows, count)) * 6.0)
    _, plan = small_plan(device)
    gb, ub = device.resident_buffer_from(g), device.resident_buffer_from(u)
    ob = device.create_resident_buffer(g.nbytes)
    plan.silu_multiply(rows, count, gb, ub, ob, limit)
    np.testing.assert_array_equal(ob.read(np.uint16).reshape(g.shape), mo.silu_multiply(g, u, limit))
    plan.residual_add(rows, count, gb, ub, ob)
    np.testing.assert_array_equal(ob.read(np.uint16).reshape(g.shape), mo.add_bf16(g, u))
    plan.destroy()


@pytest.mark.parametrize("dtype", [np.int32, np.int64])
@pytest.mark.parametrize("always", [0, 1])
def test_token_id_table_routing_is_bit_exact(device, dtype, always):
    rng = np.random.default_rng(11 + always)
    tokens, vocab, routed, k = 97, 500, 32, 4
    table = np.stack([rng.choice(routed, k, replace=False) for _ in range(vocab)]).astype(dtype)
    table[7, 1] = table[7, 0]          # a repeated index
    table[9, 2] = routed               # an index beyond the routed resources
    if dtype == np.int64:
        table[11, 0] += 1 << 32        # a non-zero high word
    token_ids = rng.integers(0, vocab, tokens).astype(np.uint32)
    token_ids[:5] = [7, 9, 11, vocab + 3, 0]
    cfg = synthetic.MoeConfig("pre", 64, 64, routed, k, router_kind=3, activation=synthetic.ACT_SIGMOID, normalize_selected=1,
                              routed_scale=2.5, always_count=always, always_weight=1.0, act_block=32)
    plan = MoePlan(device, geometry_from_config(cfg, tokens))
    rp = mo.router_params_from(cfg)
    want_tel = np.zeros(rp.telemetry_words(), dtype=np.uint32)
    want_sel, bad = mo.resource_preselect_table(token_ids, table, routed, k, always, want_tel)
    assert bad >= (4 if dtype == np.int64 else 3)
    tb = device.resident_buffer_from(token_ids)
    sb = device.create_resident_buffer(want_sel.nbytes)
    tab = device.resident_buffer_from(table)
    tel = device.create_resident_buffer(want_tel.nbytes)
    plan.parameter_table_resource_preselection(tokens, tb, sb, tab, vocab, table.dtype.itemsize // 4, tel)
    np.testing.assert_array_equal(sb.read(np.uint32).reshape(want_sel.shape), want_sel)
    np.testing.assert_array_equal(tel.read(np.uint32), want_tel)
    assert plan.status() & 2
    # the preselected router on those selections
    logits = mo.f32_to_bf16(rng.standard_normal((tokens, routed)).astype(np.float32) * 3).view(np.uint32)
    want_routes = mo.route_preselected(rp, logits, want_sel)
    lb = device.resident_buffer_from(logits)
    rb = device.create_resident_buffer(want_routes.nbytes)
    plan.moe_route_preselected(tokens, lb, sb, rb)
    np.testing.assert_array_equal(rb.read(np.uint32).reshape(want_routes.shape), want_routes)
    assert (want_routes[0] == 0x0000FFFF).all() and plan.status() & 2
    plan.destroy()


@pytest.mark.parametrize("path", [pytest.param(1, id="simt"), pytest.param(2, id="tcgen05")])
@pytest.mark.parametrize("tokens,rows,cols,block", [(1, 128, 128, 128), (40, 384, 256, 32), (120, 2880, 2880, 32)])
def test_dense_linear_matches_checker(device, path, tokens, rows, cols, block):
    rng = np.random.default_rng(tokens + rows)
    x = bf16(rng.standard_normal((tokens, cols)))
    w = rng.integers(0, 256, (rows, cols // 2), dtype=np.uint8)
    sc = rng.integers(121, 128, (rows, cols // 32), dtype=np.uint8)
    _, plan = small_plan(device, tokens=tokens, act_block=block, path=path, hidden=128 if block == 128 else 256,
                         intermediate=128 if block == 128 else 384)
    xb, wb, sb = device.resident_buffer_from(x), device.resident_buffer_from(w), device.resident_buffer_from(sc)
    ob = device.create_resident_buffer(tokens * rows * 2)
    for call in range(2):  # the second call reuses the resolved tables
        ob.fill(0)
        plan.dense_linear(tokens, xb, ob, wb, sb, rows, cols)
        assert_close(ob.read(np.uint16).reshape(tokens, rows), mo.dense_linear_mxfp4(x, w, sc, block, tier=1),
                     f"dense linear {rows}x{cols} T{tokens} path{path}")
    assert plan.status() == 0
    # new scale bytes behind the same buffer are picked up (the write bumps the record's generation)
    sc2 = rng.integers(121, 128, sc.shape, dtype=np.uint8)
    sb.write_bytes(sc2)
    plan.dense_linear(tokens, xb, ob, wb, sb, rows, cols)
    assert_close(ob.read(np.uint16).reshape(tokens, rows), mo.dense_linear_mxfp4(x, w, sc2, block, tier=1))
    plan.destroy()


def _ffn_block_nodes(hidden, intermediate, experts, k, limit):
    """The compiler's node list for one feed-forward block, resized from the committed one (4 experts of
    128 x 128) by editing exactly the attributes the compiler derives from the sizes."""
    nodes = copy.deepcopy(GOLDEN["nodes"])
    router, gate_up, down, reduce = nodes[1], nodes[2], nodes[3], nodes[4]
    router["attrs"].update(experts_per_token=k, routed_resource_count=experts, routed_selection_count=k)
    router["attrs"]["selection_domain"].update(resource_count=experts)
    router["attrs"]["selection_domain"]["encoding"].update(selection_count_per_activation=k,
                                                           index_mask=(1 << (experts - 1).bit_length()) - 1)
    for node, projections in ((gate_up, ("w1", "w3")), (down, ("w2",))):
        node["attrs"].update(hidden_size=hidden, intermediate_size=intermediate, experts_per_token=k)
        node["attrs"]["selected_parameter_accesses"][0]["mapping"] = [
            {"selector": e, "parameter_ids": [f"routed_expert_{e:03d}_{p}{s}" for p in projections for s in ("", "_scale")]}
            for e in range(experts)]
    gate_up["attrs"]["swiglu_limit"] = limit
    reduce["attrs"].update(hidden_size=hidden, experts_per_token=k)
    nodes[7]["attrs"].update(element_count=intermediate, limit=limit)
    return nodes


@pytest.mark.parametrize("path", [pytest.param(1, id="simt"), pytest.param(2, id="tcgen05")])
def test_feed_forward_block_runs_node_by_node_from_the_compilers_list(device, path):
    """ffn_norm -> the five MoE nodes -> the dense shared expert -> the add, every node through the entry
    point the dispatch list names, against the CPU checker's restatement of the same nodes."""
    hidden, intermediate, experts, k, limit, tokens = 256, 384, 8, 2, 10.0, 50
    nodes = _ffn_block_nodes(hidden, intermediate, experts, k, limit)
    dispatch = plan_from_nodes(nodes, max_tokens=tokens, selection_bias_dtype="F32", act_block=128)
    plan = MoePlan(device, dispatch.geometry)
    plan.set_expert_path(path)
    cfg = synthetic.MoeConfig("block", hidden, intermediate, experts, k, router_kind=0, activation=synthetic.ACT_SIGMOID,
                              normalize_selected=1, routed_scale=2.5, bias_dtype=synthetic.BIAS_F32, swiglu_limit=limit, act_block=128)
    case = synthetic.make_case(cfg, tokens, seed=21)
    rng = np.random.default_rng(21)
    norm_w = bf16(1.0 + 0.05 * rng.standard_normal(hidden))
    shared = {name: (rng.integers(0, 256, (r, c // 2), dtype=np.uint8), rng.integers(121, 126, (r, c // 32), dtype=np.uint8))
              for name, r, c in (("w1", intermediate, hidden), ("w3", intermediate, hidden), ("w2", hidden, intermediate))}

    # ---- CPU checker, node by node -------------------------------------------------------------
    normed = mo.rms_norm(case.hidden, norm_w, 1e-6)
    ncase = copy.copy(case)
    ncase.hidden = normed
    routed = oracle_layer(ncase, tier=1)
    gate = mo.dense_linear_mxfp4(normed, *shared["w1"], 128)
    up = mo.dense_linear_mxfp4(normed, *shared["w3"], 128)
    act = mo.silu_multiply(gate, up, limit)
    shared_out = mo.dense_linear_mxfp4(act, *shared["w2"], 128)
    want = mo.add_bf16(routed["output"], shared_out)

    # ---- the device, through the dispatch list ---------------------------------------------------
    bank = ExpertBank.upload(device, case.w1, case.s1, case.w3, case.s3, case.w2, case.s2)
    T, K = tokens, k
    buf = {
        "ffn_norm_in": device.resident_buffer_from(case.hidden),
        "ffn_norm_out": device.create_resident_buffer(T * hidden * 2),
        "moe_router": device.resident_buffer_from(case.router_w),
        "moe_router_selection_bias": device.resident_buffer_from(case.select_bias),
        "moe_router_logits": device.create_resident_buffer(T * ((experts + 1) // 2) * 4),
        "moe_routes": device.create_resident_buffer(T * K * 4),
        "moe_expert_intermediates": device.create_resident_buffer(T * plan.frame_words * 4),
        "moe_expert_outputs": device.create_resident_buffer(T * K * hidden * 2),
        "routed_moe_out": device.create_resident_buffer(T * hidden * 2),
        "shared_expert_gate": device.create_resident_buffer(T * intermediate * 2),
        "shared_expert_up": device.create_resident_buffer(T * intermediate * 2),
        "shared_expert_hidden": device.create_resident_buffer(T * intermediate * 2),
        "shared_expert_out": device.create_resident_buffer(T * hidden * 2),
        "ffn_out": device.create_resident_buffer(T * hidden * 2),
        "sparse_moe_gate_up.address_table": bank.gate_up_addresses, "sparse_moe_gate_up.parameter_slots": bank.gate_up_slots,
        "sparse_moe_down.address_table": bank.down_addresses, "sparse_moe_down.parameter_slots": bank.down_slots,
    }
    for name, (w, s) in shared.items():
        buf[f"shared_expert_{name}"] = device.resident_buffer_from(w)
        buf[f"shared_expert_{name}_scale"] = device.resident_buffer_from(s)
    plan.rms_norm(T, hidden, buf["ffn_norm_in"], buf["ffn_norm_out"], device.resident_buffer_from(norm_w), 1e-6)
    plan.run_dispatch(dispatch, T, buf)
    assert plan.status() == 0
    np.testing.assert_array_equal(buf["ffn_norm_out"].read(np.uint16).reshape(T, hidden), normed)
    np.testing.assert_array_equal(buf["moe_routes"].read(np.uint32).reshape(T, K), routed["routes"])
    assert_close(buf["routed_moe_out"].read(np.uint16).reshape(T, hidden), routed["output"], f"ffn block routed path{path}")
    assert_close(buf["shared_expert_out"].read(np.uint16).reshape(T, hidden), shared_out, f"ffn block shared expert path{path}")
    assert_close(buf["ffn_out"].read(np.uint16).reshape(T, hidden), want, f"ffn block output path{path}")
    plan.destroy()
