"""The expert-parallel layer with the collectives inside the library, on a communicator of one rank.

One rank owns every expert, sends every row to itself and must reproduce the ordinary layer call bit
for bit; the exchange code (pack into segments, grouped send/receive, preselected-route layer, unpack,
combine) is the same that several GPUs run (tests/test_gpu_expert_parallel.py needs two or four)."""
import numpy as np
import pytest

from nerve_b200 import synthetic
from nerve_b200.backend import CudaComputeDevice, ExpertBank, ExpertParallelGroup, MoePlan
from nerve_b200.expert_parallel import contiguous_owner_table

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("path", [pytest.param(1, id="simt"), pytest.param(2, id="tcgen05")])
def test_one_rank_communicator_reproduces_the_layer(path):
    cfg = synthetic.small_variant(synthetic.CONFIGS["deepseek-v3"], 256, 128, 16)  # shared expert stays local
    tokens, K, H = 20, cfg.total_k, cfg.hidden
    case = synthetic.make_case(cfg, tokens, seed=11)
    device = CudaComputeDevice(0)
    try:
        home = MoePlan.for_config(device, cfg, tokens)
        work_cfg = synthetic.MoeConfig(name="work", hidden=H, intermediate=cfg.intermediate, experts=cfg.total_experts, k=1,
                                       swiglu_limit=cfg.swiglu_limit, swiglu_alpha=cfg.swiglu_alpha,
                                       swiglu_up_offset=cfg.swiglu_up_offset, act_block=cfg.act_block)
        work = MoePlan.for_config(device, work_cfg, tokens * K)
        for plan in (home, work):
            plan.set_expert_path(path)
        bank = ExpertBank.upload(device, case.w1, case.s1, case.w3, case.s3, case.w2, case.s2)
        hidden = device.resident_buffer_from(case.hidden)
        router_w = device.resident_buffer_from(case.router_w)
        router_b = device.resident_buffer_from(case.router_bias) if case.router_bias is not None else None
        select_b = device.resident_buffer_from(case.select_bias) if case.select_bias is not None else None
        want_buf = device.create_resident_buffer(tokens * H * 2)
        home.layer(tokens, bank, hidden, want_buf, router_weights=router_w, router_bias=router_b, bias=select_b)
        want = want_buf.read(np.uint16).copy()

        owner = device.resident_buffer_from(contiguous_owner_table(cfg.total_experts, cfg.experts, 1))
        group = ExpertParallelGroup(device, ExpertParallelGroup.unique_id(), 0, 1)
        got_buf = device.create_resident_buffer(tokens * H * 2)
        for call in range(2):
            got_buf.fill(0x33)
            group.layer(home, work, tokens, bank, hidden, got_buf, owner, router_w, router_b, select_b)
            np.testing.assert_array_equal(got_buf.read(np.uint16), want, err_msg=f"call {call}")
        assert home.status() == 0 and work.status() == 0
        group.destroy()
        home.destroy()
        work.destroy()
    finally:
        device.close()
