"""Intra-expert tensor parallelism (tensor_parallel_expert): every participant computes a 128-aligned range of
the intermediate dimension, the f32 partial planes of the down projection are summed in participant order and
scaled by the route weight (nerve/model_package_physical_experts.py:98-327,
runtime-rs/shaders/distributed_sum_f32_scale_packed_bf16_to_bf16.comp:44-66). The participants run one after
another on one GPU here; what crosses between them is only the partial planes."""
import numpy as np
import pytest

from nerve_b200 import synthetic
from nerve_b200.backend import CudaComputeDevice, ExpertBank, MoePlan, ResidentBuffer, geometry_from_config
from nerve_b200.tensor_parallel import TensorParallelParticipant, finalize
from oracle import moe_oracle as mo
from tests.helpers import assert_close, oracle_layer

pytestmark = pytest.mark.gpu
PATHS = [pytest.param(1, id="simt"), pytest.param(2, id="tcgen05")]


@pytest.fixture(scope="module")
def device():
    dev = CudaComputeDevice(0)
    yield dev
    dev.close()


@pytest.mark.parametrize("path", PATHS)
@pytest.mark.parametrize("participants", [1, 2, 4])
def test_partitioned_intermediate_reproduces_the_layer(device, path, participants):
    cfg = synthetic.MoeConfig("tp", 256, 512, 8, 2, router_kind=synthetic.ROUTER_TOPK_SOFTMAX, act_block=128, swiglu_limit=7.0)
    tokens, K, H = 70, cfg.total_k, cfg.hidden
    case = synthetic.make_case(cfg, tokens, seed=13)
    want = oracle_layer(case, tier=1)
    # one device, the whole layer: routes for everyone and the result to compare with
    whole = MoePlan(device, geometry_from_config(cfg, tokens))
    whole.set_expert_path(path)
    bank = ExpertBank.upload(device, case.w1, case.s1, case.w3, case.s3, case.w2, case.s2)
    hidden = device.resident_buffer_from(case.hidden)
    rw = device.resident_buffer_from(case.router_w)
    out = device.create_resident_buffer(tokens * H * 2)
    routes = device.create_resident_buffer(tokens * K * 4)
    whole.layer(tokens, bank, hidden, out, router_weights=rw, routes_out=routes)
    single = out.read(np.uint16).reshape(tokens, H).copy()
    np.testing.assert_array_equal(routes.read(np.uint32).reshape(tokens, K), want["routes"])

    plane_bytes = tokens * K * H * 4
    planes = device.create_resident_buffer(participants * plane_bytes)
    for p in range(participants):
        part = TensorParallelParticipant(device, cfg, tokens, p, participants,
                                         lambda e: (case.w1[e], case.s1[e], case.w3[e], case.s3[e], case.w2[e], case.s2[e]), path)
        plane = ResidentBuffer.wrap(device, planes.device_address() + p * plane_bytes, plane_bytes)
        part.partial_outputs(tokens, hidden, routes, plane)
        assert part.plan.status() == 0
        part.plan.destroy()
    expert_outputs = device.create_resident_buffer(tokens * K * H * 2)
    final = device.create_resident_buffer(tokens * H * 2)
    finalize(whole, tokens, planes, routes, expert_outputs, final, participants)
    got = final.read(np.uint16).reshape(tokens, H)
    # the finaliser itself is exact arithmetic in a fixed order: bit for bit against the checker on the same planes
    host_planes = planes.read(np.float32).reshape(participants, tokens, K * H)
    want_rows = mo.sum_f32_scale_packed_bf16(host_planes, want["routes"].reshape(-1), K * H, participants, tokens, H, 16)
    np.testing.assert_array_equal(expert_outputs.read(np.uint32), want_rows)
    # and the partitioned layer equals the layer within the expert tolerance (only the order of the f32 sum differs)
    assert_close(got, want["output"], f"tensor-parallel experts x{participants} path{path}")
    if participants == 1:
        # one participant holding everything is the canonical down projection, bit for bit
        # (runtime-rs/src/vulkan_compute/mxfp4_route_native_tests.rs:427-433)
        np.testing.assert_array_equal(got, single)
    whole.destroy()
