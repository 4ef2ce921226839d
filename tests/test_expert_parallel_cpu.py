"""The expert-parallel exchange protocol over gloo, world size 2, on CPU.

The protocol code (split sizes, the three all-to-alls, the return order) is the product's
``nerve_b200.expert_parallel.exchange``; the per-rank operators are CPU stand-ins built from the
checker, so the test pins the host logic: sharded execution must reproduce the unsharded layer
bit for bit, a bad owner table is rejected, and an undersized receive buffer is an error rather
than a hang.
"""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from nerve_b200 import expert_parallel as ep  # noqa: E402
from nerve_b200 import synthetic  # noqa: E402


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


class CpuOps:
    """Stand-ins for the CUDA operators: same buffer contracts, numpy + the CPU checker."""

    def __init__(self, cfg, case, rank, world, tokens, capacity):
        import torch

        from oracle import moe_oracle as mo

        self.torch, self.mo = torch, mo
        self.cfg, self.rank, self.world, self.T = cfg, rank, world, tokens
        self.hidden = np.ascontiguousarray(case.hidden[rank * tokens:(rank + 1) * tokens])
        self.case = case
        self.owner = ep.contiguous_owner_table(cfg.total_experts, cfg.experts, world)
        self.capacity = capacity
        self.output = None

    def route(self):
        mo, cfg = self.mo, self.cfg
        logits = mo.linear_bf16(self.hidden, self.case.router_w, self.case.router_bias)
        self.routes, bad = mo.route(mo.router_params_from(cfg), logits, self.case.select_bias)
        assert bad == 0

    def pack(self):
        torch = self.torch
        K = self.cfg.total_k
        flat = self.routes.reshape(-1)
        dest = self.owner[flat & 0xFFFF].astype(np.int64)
        dest[dest == ep.UNOWNED] = self.rank
        order = np.argsort(dest, kind="stable")  # stable by owner rank, source order within
        self.send_index = np.empty_like(order)
        self.send_index[order] = np.arange(order.size)
        rows = self.hidden[order // K]
        counts = np.bincount(dest, minlength=self.world).astype(np.int32)
        return (torch.from_numpy(rows.view(np.int16).copy()), torch.from_numpy(flat[order].view(np.int32).copy()),
                torch.from_numpy(counts))

    def compute(self, recv_rows, recv_routes, n):
        mo, cfg, torch = self.mo, self.cfg, self.torch
        out = np.zeros((max(n, 1), cfg.hidden), dtype=np.uint16)
        if n == 0:
            return torch.from_numpy(out.view(np.int16))
        rows = recv_rows[:n].numpy().view(np.uint16)
        routes = recv_routes[:n].numpy().view(np.uint32).reshape(n, 1)
        p = mo.ExpertParams(cfg.hidden, cfg.intermediate, cfg.total_experts, 1, swiglu_limit=cfg.swiglu_limit,
                            swiglu_alpha=cfg.swiglu_alpha, swiglu_up_offset=cfg.swiglu_up_offset,
                            act_block=cfg.act_block, tier=1)
        weights = mo.ExpertWeights(self.case.w1, self.case.s1, self.case.w3, self.case.s3, self.case.w2, self.case.s2)
        mine = ep.owned_experts(self.owner, self.rank)
        ga, gs = weights.gate_up_tables(mine)
        da, ds = weights.down_tables(mine)
        inter = np.zeros((n, p.frame_words), dtype=np.uint32)
        control = np.array([n, 0, 0, 0, 0, 0, 0], dtype=np.uint32)
        mo.route_compact(routes, inter, control, cfg.intermediate, 1, -(-cfg.intermediate // 32), slots=gs)
        mo.gate_up(p, rows, routes, inter, ga, gs, control)
        dc = np.array([n, 0, 0, 0, 0, 0, 0], dtype=np.uint32)
        mo.route_count(routes, dc, 1, -(-cfg.hidden // 64), slots=ds)
        outs = np.zeros((n, 1, cfg.hidden), dtype=np.uint16)
        mo.down(p, inter, routes, outs, da, ds, dc)
        out[:n] = outs[:, 0]
        return torch.from_numpy(out.view(np.int16))

    def unpack_reduce(self, returned):
        cfg = self.cfg
        rows = returned.numpy().view(np.uint16)
        expert_outputs = rows[self.send_index].reshape(self.T, cfg.total_k, cfg.hidden)
        self.output = self.mo.reduce(expert_outputs, self.T, cfg.total_k, cfg.hidden, 1.0)


    # -- fixed-segment form -------------------------------------------------------------------
    def padded_ops(self):
        torch = self.torch
        S, G, H = self.T * self.cfg.total_k, self.world, self.cfg.hidden
        self.segment = S
        zeros = lambda *shape: torch.zeros(shape, dtype=torch.int16)  # noqa: E731
        return ep.PaddedExchangeOps(self.route, self.pack_padded, self.compute_padded, self.unpack_reduce_padded,
                                    zeros(G * S, H), torch.zeros(G * S, dtype=torch.int32), zeros(G * S, H))

    def pack_padded(self):
        torch, S, G = self.torch, self.segment, self.world
        rows, routes, counts = self.pack()
        rows, routes, counts = rows.numpy(), routes.numpy(), counts.numpy()
        out_rows = np.zeros((G * S, self.cfg.hidden), dtype=np.int16)
        out_routes = np.full(G * S, -1, dtype=np.int32)  # 0xffffffff
        slot_of = np.empty(rows.shape[0], dtype=np.int64)
        start = 0
        for d in range(G):
            n = int(counts[d])
            out_rows[d * S:d * S + n] = rows[start:start + n]
            out_routes[d * S:d * S + n] = routes[start:start + n]
            slot_of[start:start + n] = d * S + np.arange(n)
            start += n
        self.send_index = slot_of[self.send_index]
        return torch.from_numpy(out_rows), torch.from_numpy(out_routes)

    def compute_padded(self, recv_rows, recv_routes):
        torch = self.torch
        routes = recv_routes.numpy().view(np.uint32)
        valid = np.nonzero(routes != 0xFFFFFFFF)[0]
        out = np.zeros((routes.size, self.cfg.hidden), dtype=np.int16)
        if valid.size:
            done = self.compute(recv_rows[torch.from_numpy(valid)], recv_routes[torch.from_numpy(valid)], valid.size)
            out[valid] = done.numpy()[:valid.size]
        return torch.from_numpy(out)

    def unpack_reduce_padded(self, returned):
        self.unpack_reduce(returned)


def _worker(rank, world, port, cfg_name, small, tokens, mode, result_dir):
    import datetime
    import time

    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    try:
        cfg = synthetic.small_variant(synthetic.CONFIGS[cfg_name], *small)
        case = synthetic.make_case(cfg, tokens * world, seed=1)
        # "undersized": rank 1 alone has too small a receive buffer; "miscount": rank 0 alone announces more rows than it packed
        capacity = 1 if (mode == "undersized" and rank == 1) else tokens * cfg.total_k * world
        backend = CpuOps(cfg, case, rank, world, tokens, capacity)
        pack = backend.pack
        if mode == "miscount" and rank == 0:
            def pack():
                rows, routes, counts = backend.pack()
                counts[1] += 1000
                return rows, routes, counts
        ops = ep.ExchangeOps(backend.route, pack, backend.compute, backend.unpack_reduce, capacity)
        if mode in ("undersized", "miscount"):
            started = time.monotonic()
            try:
                ep.exchange(ops, dist)
                message = "no error"
            except RuntimeError as error:
                message = str(error)
            (Path(result_dir) / f"err{rank}.txt").write_text(f"{time.monotonic() - started:.2f}\n{message}")
            return
        if mode == "absent":
            # rank 1 never takes part in the step; rank 0 must get an error within the group's timeout, not hang
            if rank == 1:
                time.sleep(12)
                return
            started = time.monotonic()
            try:
                ep.exchange(ops, dist)
                message = "no error"
            except Exception as error:  # gloo reports the timeout as a RuntimeError or a DistBackendError
                message = f"{type(error).__name__}: {error}"
            (Path(result_dir) / f"err{rank}.txt").write_text(f"{time.monotonic() - started:.2f}\n{message}")
            return
        if mode == "padded":
            ep.exchange_padded(backend.padded_ops(), dist)
            sent = received = tokens * cfg.total_k
        else:
            sent, received = ep.exchange(ops, dist)
        np.save(Path(result_dir) / f"out{rank}.npy", backend.output)
        np.save(Path(result_dir) / f"counts{rank}.npy", np.array([sent, received]))
    finally:
        dist.destroy_process_group()


def _spawn(cfg_name, small, tokens, mode, tmp_path):
    import torch.multiprocessing as mp

    mp.spawn(_worker, args=(2, _free_port(), cfg_name, small, tokens, mode, str(tmp_path)), nprocs=2, join=True)


@pytest.mark.parametrize("mode", ["run", "padded"])
@pytest.mark.parametrize("cfg_name,small", [("gpt-oss-120b", (64, 96, 8)), ("deepseek-v3", (128, 128, 16))])
def test_sharded_layer_equals_unsharded_layer(tmp_path, cfg_name, small, mode):
    pytest.importorskip("torch")
    from oracle import moe_oracle as mo
    from tests.helpers import oracle_layer

    tokens = 6
    _spawn(cfg_name, small, tokens, mode, tmp_path)
    cfg = synthetic.small_variant(synthetic.CONFIGS[cfg_name], *small)
    case = synthetic.make_case(cfg, tokens * 2, seed=1)
    want = oracle_layer(case, tier=1)["output"]
    got = np.concatenate([np.load(tmp_path / f"out{r}.npy") for r in range(2)])
    np.testing.assert_array_equal(got, want)
    counts = [np.load(tmp_path / f"counts{r}.npy") for r in range(2)]
    assert sum(c[0] for c in counts) == sum(c[1] for c in counts) == tokens * 2 * cfg.total_k
    assert mo.lib() is not None


def _verdicts(tmp_path):
    out = {}
    for rank in range(2):
        path = tmp_path / f"err{rank}.txt"
        if path.exists():
            seconds, message = path.read_text().split("\n", 1)
            out[rank] = (float(seconds), message)
    return out


def test_undersized_receive_buffer_is_an_error_on_every_rank_not_a_hang(tmp_path):
    """Only rank 1's buffer is too small, but rank 0 must not be left waiting in the row exchange: both give
    the step up, at once."""
    pytest.importorskip("torch")
    _spawn("gpt-oss-120b", (64, 96, 8), 6, "undersized", tmp_path)
    v = _verdicts(tmp_path)
    assert "receive buffers hold" in v[1][1]
    assert "a peer rejected" in v[0][1]
    assert v[0][0] < 5 and v[1][0] < 5, "the verdict is shared, no rank waits for a timeout"


def test_split_sizes_that_do_not_match_the_packed_rows_are_rejected_everywhere(tmp_path):
    pytest.importorskip("torch")
    _spawn("gpt-oss-120b", (64, 96, 8), 6, "miscount", tmp_path)
    v = _verdicts(tmp_path)
    assert "do not describe" in v[0][1]
    assert "a peer rejected" in v[1][1] or "receive buffers hold" in v[1][1]
    assert v[0][0] < 5 and v[1][0] < 5


def test_a_rank_that_never_joins_the_step_ends_in_a_timeout_error(tmp_path):
    """Host-made failure: rank 1 sleeps through the step. Rank 0's collective ends with an error after the
    process group's timeout (8 s here) instead of blocking for good."""
    pytest.importorskip("torch")
    _spawn("gpt-oss-120b", (64, 96, 8), 6, "absent", tmp_path)
    seconds, message = _verdicts(tmp_path)[0]
    assert message != "no error" and seconds < 11, (seconds, message)


def test_owner_tables():
    table = ep.contiguous_owner_table(257, 256, 8)
    assert table[0] == 0 and table[31] == 0 and table[32] == 1 and table[255] == 7 and table[256] == ep.UNOWNED
    assert ep.owned_experts(table, 3) == list(range(96, 128)) + [256]
    ep.validate_owner_table(table, 256, 8)
    with pytest.raises(ValueError):
        ep.contiguous_owner_table(32, 30, 4)
    bad = table.copy()
    bad[5] = 9
    with pytest.raises(ValueError):
        ep.validate_owner_table(bad, 256, 8)
