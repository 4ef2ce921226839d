"""Expert-parallel MoE layer: one process per GPU, experts sharded by rank, tokens data-parallel.

The reference shards this node pair by whole-expert ownership with the hidden frame replicated
on every participant and the routed outputs collected afterwards
(nerve/physical_execution_contracts.py:690-757,
runtime-rs/src/vulkan_distributed/execution_plans.rs:1201-1205,2318-2322).  Here the same
ownership vocabulary (an owner rank per resource, contiguous ``expert_range`` by default, "every
resource owned exactly once") drives an all-to-all exchange over NCCL/NVLink instead:

    route locally -> pack routes by owner rank -> all-to-all(rows, route words)
      -> grouped gate/up + down on the owner -> all-to-all back -> unpack -> moe_reduce

Every per-route row is computed by the same kernels, on the same operands, as on one GPU, and the
combine sums them in the same order, so the result is bit-identical to the single-GPU layer.

Three forms of the same protocol:

* ``native``: the library owns the NCCL communicator and issues the two exchanges itself as grouped
  send/receive on its compute stream, fixed-size segments per peer, one C call per step
  (``nvmoe_ep_create`` / ``nvmoe_ep_layer``); torch.distributed is only used once, to hand the
  communicator id round.
* ``padded`` (:func:`exchange_padded`): the same fixed segments over ``all_to_all_single`` with equal splits.
* ``ragged`` (:func:`exchange`): rows packed back to back, split sizes read on the host.

The two torch forms are backend-neutral: the GPU path plugs in the CUDA operators, the CPU tests plug
in stand-ins and run them over gloo.
"""
from __future__ import annotations

import os
from dataclasses import dataclass

import numpy as np

UNOWNED = 0xFFFFFFFF


def contiguous_owner_table(total_experts: int, routed_experts: int, world: int) -> np.ndarray:
    """expert -> owner rank with contiguous ranges (expert_start = rank * E / G); resources past the
    routed ones (always-selected, i.e. shared experts) are replicated and stay on the token's rank."""
    if routed_experts % world:
        raise ValueError(f"{routed_experts} routed experts do not split evenly over {world} ranks")
    per = routed_experts // world
    table = np.full(total_experts, UNOWNED, dtype=np.uint32)
    table[:routed_experts] = np.arange(routed_experts, dtype=np.uint32) // per
    return table


def validate_owner_table(table: np.ndarray, routed_experts: int, world: int) -> None:
    """The reference's placement rule: every routed resource is owned exactly once, by a real rank."""
    if table.dtype != np.uint32 or table.ndim != 1 or table.size < routed_experts:
        raise ValueError("owner table must be a uint32 vector covering every resource")
    routed = table[:routed_experts]
    if np.any(routed >= world):
        raise ValueError("a routed expert has no owner among the ranks")


def owned_experts(table: np.ndarray, rank: int) -> list[int]:
    return [int(e) for e in np.nonzero((table == rank) | (table == UNOWNED))[0]]


@dataclass
class ExchangeOps:
    """What :func:`exchange` needs from a backend. Tensors are torch tensors on the backend's device."""

    route: callable        # () -> None: fills the local routes
    pack: callable         # () -> (send_rows [R,H] int16, send_routes [R] int32, dest_counts [G] int32)
    compute: callable      # (recv_rows [N,H], recv_routes [N], n) -> rows [N,H] int16 (first n valid)
    unpack_reduce: callable  # (returned_rows [R,H]) -> None: fills the output
    capacity: int          # rows the receive buffers hold


def exchange(ops: ExchangeOps, dist, group=None):
    """One layer step of the all-to-all protocol. Returns (rows sent, rows received)."""
    import torch

    ops.route()
    send_rows, send_routes, dest_counts = ops.pack()
    world = dist.get_world_size(group)
    # split sizes travel first; they are needed on the host to size the row exchange
    recv_counts = torch.empty_like(dest_counts)
    dist.all_to_all_single(recv_counts, dest_counts, group=group)
    send_splits = [int(v) for v in dest_counts.cpu().tolist()]
    recv_splits = [int(v) for v in recv_counts.cpu().tolist()]
    n_send, n_recv = sum(send_splits), sum(recv_splits)
    problem = None
    if len(send_splits) != world or min(send_splits, default=0) < 0 or n_send > send_rows.shape[0]:
        problem = f"destination counts {send_splits} do not describe {send_rows.shape[0]} packed rows"
    elif min(recv_splits, default=0) < 0:
        problem = f"a peer announced a negative row count: {recv_splits}"
    elif n_recv > ops.capacity:
        problem = f"{n_recv} rows arrive but the receive buffers hold {ops.capacity}"
    # A rank that found a problem must not simply leave: its peers would wait in the row exchange for rows that
    # never come. The verdicts are shared first (one small all-reduce beside a host read that the split sizes
    # need anyway), and every rank gives the step up together.
    verdict = dest_counts.new_tensor([0 if problem is None else 1])
    dist.all_reduce(verdict, op=dist.ReduceOp.MAX, group=group)
    if problem is not None:
        raise RuntimeError(problem)
    if int(verdict.cpu().item()) != 0:
        raise RuntimeError("a peer rejected this step's split sizes: the exchange was given up on every rank")
    hidden = send_rows.shape[1]
    recv_rows = torch.empty((max(n_recv, 1), hidden), dtype=send_rows.dtype, device=send_rows.device)
    recv_routes = torch.empty((max(n_recv, 1),), dtype=send_routes.dtype, device=send_routes.device)
    # bf16 rows travel as pairs in 32-bit words (every backend moves int32; gloo has no 16-bit all-to-all)
    as_words = lambda t: t.view(torch.int32)  # noqa: E731
    dist.all_to_all_single(as_words(recv_rows)[:n_recv], as_words(send_rows)[:n_send], recv_splits, send_splits, group=group)
    dist.all_to_all_single(recv_routes[:n_recv], send_routes[:n_send], recv_splits, send_splits, group=group)
    done = ops.compute(recv_rows, recv_routes, n_recv)
    returned = torch.empty((max(n_send, 1), hidden), dtype=send_rows.dtype, device=send_rows.device)
    dist.all_to_all_single(as_words(returned)[:n_send], as_words(done)[:n_recv], send_splits, recv_splits, group=group)
    ops.unpack_reduce(returned)
    return n_send, n_recv


@dataclass
class PaddedExchangeOps:
    """What :func:`exchange_padded` needs from a backend: every buffer has ``world * segment_rows`` rows,
    segment ``d`` holding what goes to (or came from) rank ``d``; unused slots carry the route word
    0xffffffff. All tensors are allocated once by the backend."""

    route: callable          # () -> None
    pack: callable           # () -> (send_rows [G*S,H] int16, send_routes [G*S] int32)
    compute: callable        # (recv_rows, recv_routes) -> rows [G*S,H] int16, slot for slot
    unpack_reduce: callable  # (returned_rows [G*S,H]) -> None
    recv_rows: object
    recv_routes: object
    returned: object


def exchange_padded(ops: PaddedExchangeOps, dist, group=None):
    """One layer step with fixed-size segments: three equal-split all-to-alls and no host read in between
    (for decode-sized batches, where shipping the unused slots costs less than a device-to-host sync)."""
    import torch

    ops.route()
    send_rows, send_routes = ops.pack()
    as_words = lambda t: t.view(torch.int32)  # noqa: E731
    dist.all_to_all_single(as_words(ops.recv_rows), as_words(send_rows), group=group)
    dist.all_to_all_single(ops.recv_routes, send_routes, group=group)
    done = ops.compute(ops.recv_rows, ops.recv_routes)
    dist.all_to_all_single(as_words(ops.returned), as_words(done), group=group)
    ops.unpack_reduce(ops.returned)


PADDED_EXCHANGE_LIMIT_BYTES = 64 << 20  # send buffer size up to which fixed segments beat a host sync


class ExpertParallelLayer:
    """The GPU backend of :func:`exchange` / :func:`exchange_padded` for one rank."""

    def __init__(self, cfg, tokens_per_rank: int, rank: int, world: int, device_index: int, seed: int = 0,
                 owner_table: np.ndarray | None = None, expert_path: int = 0, mode: str = "auto", banks: int = 1,
                 dist=None, capacity_factor: float = 0.0):
        """mode: "native" = the library issues the collectives itself (one call per step, needs `dist` once to
        hand the communicator id round); "padded" / "ragged" = the same protocol over torch.distributed with
        fixed segments / with split sizes read on the host; "auto" = native when `dist` is given and the
        fixed segments are small enough, else padded or ragged by size.
        capacity_factor (native form): the segment a rank keeps for each peer holds this many times the mean
        number of rows per peer (tokens * top_k / world), instead of the worst case tokens * top_k; 0 = worst
        case. A step whose routing overflows a segment raises NVMOE_STATUS_EXCHANGE_OVERFLOW (`overflowed()`)."""
        import torch

        from . import synthetic
        from .backend import CudaComputeDevice, MoePlan, ResidentBuffer
        from .resident_layer import upload_expert_banks

        self.torch = torch
        self.cfg, self.rank, self.world, self.tokens = cfg, rank, world, tokens_per_rank
        self.owner = contiguous_owner_table(cfg.total_experts, cfg.experts, world) if owner_table is None else owner_table
        validate_owner_table(self.owner, cfg.experts, world)
        torch.cuda.set_device(device_index)
        self.tdev = torch.device("cuda", device_index)
        self.device = CudaComputeDevice(device_index)
        # kernels and collectives are ordered by one stream: a torch stream of our own (torch's default
        # stream has handle 0, which the library reads as "use your own stream"), current during step()
        self.stream = torch.cuda.Stream(device=self.tdev)
        self.device.set_stream(self.stream.cuda_stream)
        T, K, H, G = tokens_per_rank, cfg.total_k, cfg.hidden, world
        bounded = T * K  # the most rows one rank can be sent by one peer
        if capacity_factor > 0.0 and G > 1:
            eights = -(-int(np.ceil(capacity_factor * T * K / G)) // 8) * 8  # whole groups of eight rows
            bounded = max(8, min(T * K, eights))
        if mode == "auto":
            mode = os.environ.get("NVMOE_EP_MODE", "auto")
        if mode == "auto":
            small = bounded * G * H * 2 <= PADDED_EXCHANGE_LIMIT_BYTES
            mode = ("native" if dist is not None else "padded") if small else "ragged"
        if mode not in ("native", "padded", "ragged"):
            raise ValueError(f"unknown exchange mode {mode!r}")
        if mode == "native" and dist is None:
            raise ValueError("the native exchange needs torch.distributed once, to share the communicator id")
        self.mode = mode
        # the fixed-segment forms may bound their segments; the ragged form sizes its receive buffer for the worst case
        self.segment = bounded if mode in ("native", "padded") else T * K
        self.capacity_factor = capacity_factor if self.segment < T * K else 0.0
        self.capacity = self.segment * G
        # this rank's tokens: rank r owns tokens [r*T, (r+1)*T) of the global batch
        case = synthetic.make_case(cfg, T * G, seed=seed, with_weights=False)
        self.case = case
        local = slice(rank * T, (rank + 1) * T)
        self.hidden_host = np.ascontiguousarray(case.hidden[local])
        mine = owned_experts(self.owner, rank)
        # `banks` resident copies of this rank's experts, used in turn (a benchmark's way of keeping the
        # weights of a step out of L2, as the other layers of a model would)
        self.banks = upload_expert_banks(self.device, cfg, seed, set(mine), max(1, banks))
        self.bank = self.banks[0]
        self.turn = 0
        self.home = MoePlan.for_config(self.device, cfg, T)
        work_cfg = synthetic.MoeConfig(
            cfg.name + "-work", cfg.hidden, cfg.intermediate, cfg.total_experts, 1, swiglu_limit=cfg.swiglu_limit,
            swiglu_alpha=cfg.swiglu_alpha, swiglu_up_offset=cfg.swiglu_up_offset, act_block=cfg.act_block)
        self.work = MoePlan.for_config(self.device, work_cfg, self.capacity)
        for plan in (self.home, self.work):
            if expert_path:
                plan.set_expert_path(expert_path)

        def dev_tensor(shape, dtype):
            return torch.zeros(shape, dtype=dtype, device=self.tdev)

        def wrap(t):
            return ResidentBuffer.wrap(self.device, t.data_ptr(), t.numel() * t.element_size())

        i16, i32 = torch.int16, torch.int32
        self.t_hidden = torch.from_numpy(self.hidden_host.view(np.int16)).to(self.tdev)
        self.t_router_w = torch.from_numpy(case.router_w.view(np.int16)).to(self.tdev)
        self.t_logits = dev_tensor((T, (cfg.experts + 1) // 2), i32)
        self.t_routes = dev_tensor((T, K), i32)
        send_slots = self.capacity if self.mode == "padded" else T * K
        self.t_send_rows = dev_tensor((send_slots, H), i16)
        self.t_send_routes = dev_tensor((send_slots,), i32)
        self.t_send_index = dev_tensor((T * K,), i32)
        self.t_dest_counts = dev_tensor((G,), i32)
        self.t_owner = torch.from_numpy(self.owner.view(np.int32)).to(self.tdev)
        self.t_frames = dev_tensor((self.capacity, self.work.frame_words), i32)
        self.t_work_out = dev_tensor((self.capacity, H), i16)
        self.t_controls = dev_tensor((16,), i32)
        self.t_expert_outputs = dev_tensor((T, K, H), i16)
        self.t_output = dev_tensor((T, H), i16)
        self.b = {name: wrap(getattr(self, "t_" + name)) for name in (
            "hidden", "router_w", "logits", "routes", "send_rows", "send_routes", "send_index", "dest_counts",
            "owner", "frames", "work_out", "expert_outputs", "output")}
        self.b["gate_control"] = ResidentBuffer.wrap(self.device, self.t_controls.data_ptr(), 28)
        self.b["down_control"] = ResidentBuffer.wrap(self.device, self.t_controls.data_ptr() + 32, 28)
        self.router_bias = self.device.resident_buffer_from(case.router_bias) if case.router_bias is not None else None
        self.select_bias = self.device.resident_buffer_from(case.select_bias) if case.select_bias is not None else None
        self.telemetry = self.device.create_resident_buffer(self.home.telemetry_words() * 4)
        self.ops = ExchangeOps(self._route, self._pack, self._compute, self._unpack_reduce, self.capacity)
        torch.cuda.synchronize(self.tdev)  # the buffers above were filled on torch's default stream
        if self.mode == "native":
            from .backend import ExpertParallelGroup

            id_bytes = torch.zeros(128, dtype=torch.uint8, device=self.tdev)
            if rank == 0:
                id_bytes.copy_(torch.frombuffer(bytearray(ExpertParallelGroup.unique_id()), dtype=torch.uint8))
            dist.broadcast(id_bytes, 0)
            self.group = ExpertParallelGroup(self.device, bytes(id_bytes.cpu().numpy().tobytes()), rank, world)
        if self.mode == "padded":
            self.t_recv_rows = dev_tensor((self.capacity, H), i16)
            self.t_recv_routes = dev_tensor((self.capacity,), i32)
            self.t_returned = dev_tensor((self.capacity, H), i16)
            for name in ("recv_rows", "recv_routes", "returned"):
                self.b[name] = wrap(getattr(self, "t_" + name))
            self.padded_ops = PaddedExchangeOps(self._route, self._pack_padded, self._compute_padded,
                                                self._unpack_reduce_padded, self.t_recv_rows, self.t_recv_routes,
                                                self.t_returned)

    # -- backend pieces ------------------------------------------------------------------------
    def _route(self):
        b, T = self.b, self.tokens
        self.home.linear(T, b["hidden"], b["logits"], b["router_w"], self.router_bias)
        self.home.moe_route(T, b["logits"], b["routes"], self.select_bias, self.telemetry)

    def _pack(self):
        b = self.b
        self.home.ep_pack(self.tokens, b["hidden"], b["routes"], b["owner"], self.world, self.rank, b["send_rows"],
                          b["send_routes"], b["send_index"], b["dest_counts"])
        return self.t_send_rows, self.t_send_routes, self.t_dest_counts

    def _compute(self, recv_rows, recv_routes, n):
        from .backend import ResidentBuffer

        if n == 0:
            return self.t_work_out
        b = self.b
        rows = ResidentBuffer.wrap(self.device, recv_rows.data_ptr(), n * recv_rows.shape[1] * 2)
        routes = ResidentBuffer.wrap(self.device, recv_routes.data_ptr(), n * 4)
        control = self.torch.tensor([n, 0, 0, 0, 0, 0, 0, 0, n, 0, 0, 0, 0, 0, 0, 0], dtype=self.torch.int32)
        self.t_controls.copy_(control, non_blocking=False)
        w = self.work
        w.moe_route_compact(n, routes, b["frames"], b["gate_control"], self.bank.gate_up_slots)
        w.independent_sparse_moe_gate_up(n, rows, routes, b["frames"], self.bank.gate_up_addresses,
                                         self.bank.gate_up_slots, b["gate_control"])
        w.moe_route_count(n, routes, b["down_control"], self.bank.down_slots)
        w.independent_sparse_moe_down(n, b["frames"], routes, b["work_out"], self.bank.down_addresses,
                                      self.bank.down_slots, b["down_control"])
        rows.destroy()
        routes.destroy()
        return self.t_work_out

    def _unpack_reduce(self, returned):
        from .backend import ResidentBuffer

        T = self.tokens
        rb = ResidentBuffer.wrap(self.device, returned.data_ptr(), returned.numel() * 2)
        if returned.shape[0] < T * self.cfg.total_k:
            raise RuntimeError("fewer rows came back than routes were sent: a route had no owner")
        self.home.ep_unpack(T, rb, self.b["send_index"], self.b["expert_outputs"])
        self.home.moe_reduce(T, self.b["expert_outputs"], self.b["output"])
        rb.destroy()

    # -- fixed-segment form: nothing is read on the host between the kernels ------------------------
    def _pack_padded(self):
        b = self.b
        self.home.ep_pack(self.tokens, b["hidden"], b["routes"], b["owner"], self.world, self.rank, b["send_rows"],
                          b["send_routes"], b["send_index"], b["dest_counts"], segment_rows=self.segment)
        return self.t_send_rows, self.t_send_routes

    def _compute_padded(self, recv_rows, recv_routes):
        # the owner's side of the layer on preselected routes: every resource in range, the slot tables
        # (unbound for experts of other ranks) keep what this rank owns; padding slots name expert 0xffff
        b = self.b
        self.work.layer(self.capacity, self.bank, b["recv_rows"], None, routes_in=b["recv_routes"],
                        expert_outputs=b["work_out"], expert_start=0, expert_count=self.cfg.total_experts)
        return self.t_work_out

    def _unpack_reduce_padded(self, returned):
        self.home.ep_unpack(self.tokens, self.b["returned"], self.b["send_index"], self.b["expert_outputs"])
        self.home.moe_reduce(self.tokens, self.b["expert_outputs"], self.b["output"])

    def step(self, dist, group=None):
        self.turn += 1
        self.bank = self.banks[self.turn % len(self.banks)]
        if self.mode == "native":
            b = self.b
            self.group.layer(self.home, self.work, self.tokens, self.bank, b["hidden"], b["output"], b["owner"],
                             b["router_w"], self.router_bias, self.select_bias, self.telemetry,
                             capacity_rows=self.segment if self.segment < self.tokens * self.cfg.total_k else 0)
            return self.tokens * self.cfg.total_k, -1
        with self.torch.cuda.stream(self.stream):
            if self.mode == "padded":
                exchange_padded(self.padded_ops, dist, group)
                return self.tokens * self.cfg.total_k, -1
            return exchange(self.ops, dist, group)

    def output(self) -> np.ndarray:
        self.torch.cuda.synchronize()
        return self.t_output.cpu().numpy().view(np.uint16)

    def overflowed(self) -> bool:
        """Whether a step since the last call left routes out because a capacity-bounded segment was full
        (reads and clears the plan's status word: synchronises)."""
        return bool(self.home.status() & 16)
