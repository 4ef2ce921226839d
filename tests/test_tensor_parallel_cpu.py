"""Host logic of the tensor-parallel expert split, without a GPU: the 128-aligned ranges, and that the
participants' weight slices partition the layer (the checker's down projection over each slice, summed in
participant order and finalised, gives the unpartitioned result up to the order of the f32 sum)."""
import numpy as np
import pytest

from nerve_b200 import synthetic
from nerve_b200.tensor_parallel import intermediate_ranges, slice_expert_tensors
from oracle import moe_oracle as mo
from tests.helpers import assert_close, expert_params, oracle_layer


def test_ranges_are_whole_blocks():
    assert intermediate_ranges(2048, 8) == [(i * 256, 256) for i in range(8)]
    assert intermediate_ranges(512, 1) == [(0, 512)]
    with pytest.raises(ValueError):
        intermediate_ranges(2880, 4)  # 720 columns are not whole 128-blocks


@pytest.mark.parametrize("participants", [2, 4])
def test_slices_partition_the_layer(participants):
    cfg = synthetic.MoeConfig("tp", 128, 512, 4, 2, router_kind=synthetic.ROUTER_TOPK_SOFTMAX, act_block=128, swiglu_limit=7.0)
    tokens, K, H = 9, cfg.total_k, cfg.hidden
    case = synthetic.make_case(cfg, tokens, seed=3)
    want = oracle_layer(case, tier=1)
    routes = want["routes"]
    planes = np.zeros((participants, tokens, K * H), dtype=np.float32)
    for p, (start, count) in enumerate(intermediate_ranges(cfg.intermediate, participants)):
        local = synthetic.replace(cfg, intermediate=count)
        sliced = [slice_expert_tensors((case.w1[e], case.s1[e], case.w3[e], case.s3[e], case.w2[e], case.s2[e]), start, count)
                  for e in range(cfg.total_experts)]
        weights = mo.ExpertWeights(*[[s[i] for s in sliced] for i in range(6)])
        ep = expert_params(local, tier=1)
        inter = np.zeros((tokens, ep.frame_words), dtype=np.uint32)
        control = np.array([tokens, 0, 0, 0, 0, 0, 0], dtype=np.uint32)
        ga, gs = weights.gate_up_tables()
        mo.route_compact(routes, inter, control, count, K, -(-count // 32))
        mo.gate_up(ep, case.hidden, routes, inter, ga, gs, control)
        # the participant's slice of the intermediates is the matching columns of the unpartitioned ones
        full = want["intermediates"][:, : K * cfg.intermediate // 2].view(np.uint16).reshape(tokens, K, cfg.intermediate)
        mine = inter[:, : K * count // 2].view(np.uint16).reshape(tokens, K, count)
        np.testing.assert_array_equal(mine, full[:, :, start:start + count])
        # partial planes: the down projection with unit route weights is the raw sum (rounded to bf16 here, which
        # is enough to check the partition; the device keeps f32)
        unit = (routes & 0xFFFF) | (0x3F80 << 16)
        da, ds = weights.down_tables()
        outs = np.zeros((tokens, K, H), dtype=np.uint16)
        mo.down(ep, inter, unit, outs, da, ds, control)
        planes[p] = mo.bf16_to_f32(outs).reshape(tokens, K * H)
    rows = mo.sum_f32_scale_packed_bf16(planes, routes.reshape(-1), K * H, participants, tokens, H, 16)
    got = mo.reduce(rows.view(np.uint16).reshape(tokens, K, H), tokens, K, H)
    m = assert_close(got, want["output"])
    assert m["rel_l2"] < 5e-3
