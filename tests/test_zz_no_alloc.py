"""The route scheduler entry that allocates nothing on the device (fixed scratch array in the library).

Collected last on purpose: it has to pass alone and after every other GPU test has used the same
device, plans and scratch.  Checked against nvmoe_route_compact, the entry it is a variant of, against
the CPU checker's scheduler, and for leaving the device's free memory exactly as it found it.
"""
import numpy as np
import pytest

from nerve_b200 import synthetic
from nerve_b200.backend import CudaComputeDevice, CudaError, MoePlan, geometry_from_config
from oracle import moe_oracle as mo

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def device():
    dev = CudaComputeDevice(0)
    yield dev
    dev.close()


def _cfg(experts, K, intermediate):
    return synthetic.MoeConfig(name="t", hidden=64, intermediate=intermediate, experts=experts, k=K, act_block=32)


def _routes(rng, tokens, K, experts):
    ids = np.stack([np.sort(rng.choice(experts, K, replace=False)) for _ in range(tokens)]).astype(np.uint32)
    w = synthetic.f32_to_bf16(rng.random((tokens, K), dtype=np.float32)).astype(np.uint32)
    return (w << 16) | ids


def _run(device, plan, entry, tokens, routes, control_words, slots=None):
    rb = device.resident_buffer_from(routes)
    ib = device.create_resident_buffer(tokens * plan.frame_words * 4)
    ib.fill(0)
    cb = device.resident_buffer_from(np.array(control_words, dtype=np.uint32))
    sb = device.resident_buffer_from(slots) if slots is not None else None
    getattr(plan, entry)(tokens, rb, ib, cb, sb)
    device.synchronize()
    out = ib.read(np.uint32).reshape(tokens, plan.frame_words).copy(), cb.read(np.uint32).copy()
    for b in (rb, ib, cb, sb):
        if b is not None:
            b.destroy()
    return out


# (tokens, K, experts): single-block sort (no scratch), multi-block sort, many buckets
@pytest.mark.parametrize("tokens,K,experts", [(64, 4, 32), (2048, 4, 32), (2500, 9, 257)])
def test_static_scratch_entry_matches_route_compact_twice_in_a_row(device, tokens, K, experts):
    rng = np.random.default_rng(1000 + tokens)
    plan = MoePlan(device, geometry_from_config(_cfg(experts, K, 32), tokens))
    for call in range(2):  # the second call reuses the array the first one left dirty
        routes = _routes(rng, tokens, K, experts)
        want_frames, want_control = _run(device, plan, "moe_route_compact", tokens, routes, [tokens, 0, 0, 0, 0, 0, 0])
        got_frames, got_control = _run(device, plan, "moe_route_compact_static", tokens, routes, [tokens, 0, 0, 0, 0, 0, 0])
        np.testing.assert_array_equal(got_frames, want_frames, err_msg=f"call {call}")
        np.testing.assert_array_equal(got_control, want_control, err_msg=f"call {call}")
        assert want_control[3] == tokens * K
        # and both equal the checker's restatement of the scheduler shader
        oracle_frames = np.zeros((tokens, plan.frame_words), dtype=np.uint32)
        oracle_control = np.array([tokens, 0, 0, 0, 0, 0, 0], dtype=np.uint32)
        mo.route_compact(routes, oracle_frames, oracle_control, 32, K, 1)
        np.testing.assert_array_equal(got_frames, oracle_frames, err_msg=f"call {call} vs checker")
        np.testing.assert_array_equal(got_control, oracle_control, err_msg=f"call {call} vs checker")
    plan.destroy()


def test_static_scratch_entry_leaves_free_device_memory_unchanged(device):
    """The point of the entry: a caller that has given all free device memory away can still call it.
    After one warm-up call (which loads the kernels and looks the array's address up) a call must not move
    the device's free-memory figure by a single byte."""
    import torch

    tokens, K, experts = 2048, 4, 32  # the multi-block sort, the form that needs scratch
    rng = np.random.default_rng(77)
    plan = MoePlan(device, geometry_from_config(_cfg(experts, K, 32), tokens))
    routes = _routes(rng, tokens, K, experts)
    rb = device.resident_buffer_from(routes)
    ib = device.create_resident_buffer(tokens * plan.frame_words * 4)
    cb = device.resident_buffer_from(np.array([tokens, 0, 0, 0, 0, 0, 0], dtype=np.uint32))
    plan.moe_route_compact_static(tokens, rb, ib, cb)  # warm-up
    device.synchronize()
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info(device.ordinal)
    for _ in range(3):
        cb.write_bytes(np.array([tokens, 0, 0, 0, 0, 0, 0], dtype=np.uint32))
        plan.moe_route_compact_static(tokens, rb, ib, cb)
        device.synchronize()
    free_after, _ = torch.cuda.mem_get_info(device.ordinal)
    assert free_after == free_before, (free_before, free_after)
    for b in (rb, ib, cb):
        b.destroy()
    plan.destroy()


def test_static_scratch_entry_partitioned_mode(device):
    tokens, K, experts = 1500, 4, 32
    rng = np.random.default_rng(5)
    plan = MoePlan(device, geometry_from_config(_cfg(experts, K, 32), tokens))
    slots = np.full(experts * 4, 0xFFFFFFFF, dtype=np.uint32)
    for e in range(8, 20):
        if e % 3:
            slots[e * 4: e * 4 + 4] = e
    for call in range(2):
        routes = _routes(rng, tokens, K, experts)
        control = [tokens, 8, 12, 0, 0, 0, 0]
        want = _run(device, plan, "moe_route_compact", tokens, routes, control, slots)
        got = _run(device, plan, "moe_route_compact_static", tokens, routes, control, slots)
        np.testing.assert_array_equal(got[0], want[0])
        np.testing.assert_array_equal(got[1], want[1])
    plan.destroy()


def test_static_scratch_entry_rejects_sizes_beyond_the_fixed_array(device):
    # 300 000 routes in 1172 blocks x 257 buckets = 301 204 histogram words > 65 536
    tokens, K, experts = 37500, 8, 256
    plan = MoePlan(device, geometry_from_config(_cfg(experts, K, 32), tokens))
    rb = device.create_resident_buffer(tokens * K * 4)
    ib = device.create_resident_buffer(tokens * plan.frame_words * 4)
    cb = device.resident_buffer_from(np.array([tokens, 0, 0, 0, 0, 0, 0], dtype=np.uint32))
    with pytest.raises(CudaError, match="exceed the fixed scratch"):
        plan.moe_route_compact_static(tokens, rb, ib, cb)
    plan.destroy()
