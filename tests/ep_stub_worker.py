"""One-rank run of the expert-parallel layer over a stand-in NCCL (tests/stub_nccl.c), started by
test_gpu_ep_failures.py in a process that has no real NCCL loaded. Checks, from the host and without any GPU
fault: the step over the stand-in equals the plain layer; a send that fails inside the first exchange leaves
every group closed, still posts the return exchange and reports the error; the communicator keeps working
afterwards; a bounded wait that runs out, or an asynchronous error, aborts the communicator and later calls
are refused. Exit code 0 = all of it held."""
import ctypes
import sys
from pathlib import Path

import numpy as np

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))


def main() -> int:
    stub = ctypes.CDLL(sys.argv[1])
    from nerve_b200 import capi, synthetic
    from nerve_b200.backend import CudaComputeDevice, CudaError, ExpertBank, MoePlan

    assert "torch" not in sys.modules, "a framework's NCCL would be bound instead of the stand-in"
    lib = capi.load()
    cfg = synthetic.MoeConfig(name="ep-stub", hidden=256, intermediate=256, experts=8, k=2, act_block=32, swiglu_limit=7.0)
    tokens = 20
    case = synthetic.make_case(cfg, tokens, seed=2)
    device = CudaComputeDevice(0)
    home = MoePlan.for_config(device, cfg, tokens)
    work_cfg = synthetic.MoeConfig(name="work", hidden=cfg.hidden, intermediate=cfg.intermediate, experts=cfg.total_experts, k=1,
                                   swiglu_limit=cfg.swiglu_limit, act_block=cfg.act_block)
    work = MoePlan.for_config(device, work_cfg, tokens * cfg.total_k)
    bank = ExpertBank.upload(device, case.w1, case.s1, case.w3, case.s3, case.w2, case.s2)
    hidden = device.resident_buffer_from(case.hidden)
    rw = device.resident_buffer_from(case.router_w)
    owner = device.resident_buffer_from(np.zeros(cfg.total_experts, dtype=np.uint32))
    want_buf = device.create_resident_buffer(tokens * cfg.hidden * 2)
    home.layer(tokens, bank, hidden, want_buf, router_weights=rw)
    want = want_buf.read(np.uint16).copy()

    id_buf = ctypes.create_string_buffer(128)
    assert lib.nvmoe_ep_unique_id(id_buf) == 0
    handle = ctypes.c_void_p()
    device._check(lib.nvmoe_ep_create(device._h, id_buf.raw, 0, 1, ctypes.byref(handle)))
    out = device.create_resident_buffer(tokens * cfg.hidden * 2)
    args = capi.EpLayerArgs()
    args.batch_width = tokens
    args.hidden, args.output, args.owner_table, args.router_weights = hidden._h, out._h, owner._h, rw._h
    args.gate_up_addresses, args.gate_up_slots = bank.gate_up_addresses._h, bank.gate_up_slots._h
    args.down_addresses, args.down_slots = bank.down_addresses._h, bank.down_slots._h

    def counters():
        c = (ctypes.c_int * 8)()
        stub.stub_nccl_counters(c)
        return dict(zip(("group_start", "group_end", "send", "recv", "abort", "async_poll", "destroy"), list(c)))

    def step():
        return lib.nvmoe_ep_layer(handle, home._h, work._h, ctypes.byref(args))

    # 1. the step over the stand-in is the plain layer
    stub.stub_nccl_reset()
    assert step() == 0, lib.nvmoe_last_error(device._h)
    np.testing.assert_array_equal(out.read(np.uint16), want)
    c = counters()
    assert c["group_start"] == c["group_end"] == 2 and c["send"] == c["recv"] == 3, c

    # 2. a send fails inside the first exchange: the error is reported, both groups were opened and closed
    stub.stub_nccl_reset()
    stub.stub_nccl_fail_send_in(0)
    rc = step()
    assert rc == capi.ERR_COLLECTIVE, rc
    assert b"injected send failure" in lib.nvmoe_last_error(device._h)
    c = counters()
    assert c["group_start"] == 2 and c["group_end"] == 2, f"every opened group must be closed and the return exchange posted: {c}"
    device.synchronize()

    # 3. the same with the failure in the return exchange
    stub.stub_nccl_reset()
    stub.stub_nccl_fail_send_in(2)
    assert step() == capi.ERR_COLLECTIVE
    c = counters()
    assert c["group_start"] == 2 and c["group_end"] == 2, c
    device.synchronize()

    # 4. the communicator still works
    stub.stub_nccl_reset()
    out.fill(0)
    assert step() == 0
    np.testing.assert_array_equal(out.read(np.uint16), want)
    assert lib.nvmoe_ep_sync(handle, 30_000_000_000) == 0

    # 5. an asynchronous error seen while work is still queued aborts the communicator; later calls are refused
    stub.stub_nccl_reset()
    stub.stub_nccl_set_async_error(1)
    for _ in range(300):
        assert step() == 0
    rc = lib.nvmoe_ep_sync(handle, 30_000_000_000)
    c = counters()
    if rc == 0:
        # the device drained before the first poll: nothing to abort, nothing asked
        assert c["abort"] == 0
    else:
        assert rc == capi.ERR_COLLECTIVE and c["abort"] == 1 and c["async_poll"] >= 1, (rc, c)
        assert step() == capi.ERR_COLLECTIVE and b"aborted" in lib.nvmoe_last_error(device._h)
    device.synchronize()  # the queued kernels themselves were healthy: the stream drains
    lib.nvmoe_ep_destroy(handle)

    # 6. a bounded wait that runs out aborts too
    handle2 = ctypes.c_void_p()
    stub.stub_nccl_reset()
    device._check(lib.nvmoe_ep_create(device._h, id_buf.raw, 0, 1, ctypes.byref(handle2)))
    handle_save = handle
    handle = handle2
    for _ in range(300):
        assert step() == 0
    rc = lib.nvmoe_ep_sync(handle2, 1)  # one nanosecond
    c = counters()
    assert rc in (0, capi.ERR_TIMEOUT), rc
    if rc == capi.ERR_TIMEOUT:
        assert c["abort"] == 1 and b"did not finish" in lib.nvmoe_last_error(device._h)
    device.synchronize()
    lib.nvmoe_ep_destroy(handle2)
    del handle_save
    try:
        device.close()
    except CudaError:
        return 1
    print("ep stub worker: all checks held", counters())
    return 0


if __name__ == "__main__":
    sys.exit(main())
