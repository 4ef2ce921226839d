"""Host-side mirror of the reference's device object model for the MoE operators.

The reference drives its kernels through ``VulkanComputeDevice`` / ``VulkanResidentBuffer`` /
resident kernel dispatches (runtime-rs/src/vulkan_compute/compute_device_dispatch.rs:2-273,
resident_buffers.rs:39-232) with the per-operator binding order of
runtime-rs/src/vulkan_stream_circuit/circuit_binding_builder.rs:1-96.  This module keeps those
names, argument meanings and error behaviour (eager validation errors carrying a message, the way
``VulkanError(String)`` does) on top of the C ABI, so tests written against it read like the
reference's own conformance tests (runtime-rs/src/vulkan_compute/mxfp4_tests.rs).

Everything here calls the CUDA library; nothing computes on the host.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import numpy as np

from . import capi
from .synthetic import MoeConfig

UNBOUND_PARAMETER_SLOT = 0xFFFFFFFF


class CudaError(RuntimeError):
    """Counterpart of the reference's ``VulkanError(pub String)``."""

    def __init__(self, code: int, message: str):
        super().__init__(f"[{code}] {message}")
        self.code = code
        self.message = message


def _ptr(array: np.ndarray):
    return array.ctypes.data_as(ctypes.c_void_p)


class CudaComputeDevice:
    """``VulkanComputeDevice`` for one CUDA ordinal. Not thread-safe, like the reference's."""

    def __init__(self, ordinal: int = 0):
        self._lib = capi.load()
        handle = ctypes.c_void_p()
        rc = self._lib.nvmoe_device_open(ordinal, ctypes.byref(handle))
        if rc != 0:
            raise CudaError(rc, self._lib.nvmoe_last_error(None).decode())
        self._h = handle
        self.ordinal = ordinal

    def _check(self, rc: int) -> None:
        if rc != 0:
            raise CudaError(rc, self._lib.nvmoe_last_error(self._h).decode())

    def create_resident_buffer(self, byte_capacity: int) -> "ResidentBuffer":
        return ResidentBuffer(self, byte_capacity)

    def resident_buffer_from(self, array: np.ndarray) -> "ResidentBuffer":
        array = np.ascontiguousarray(array)
        buf = ResidentBuffer(self, max(array.nbytes, 1))
        if array.nbytes:
            buf.write_bytes(array)
        return buf

    def stream(self) -> int:
        """The ``cudaStream_t`` all launches of this device go to, as an integer."""
        return int(self._lib.nvmoe_device_stream(self._h) or 0)

    def set_stream(self, cuda_stream: int) -> None:
        """Launch on a stream the caller owns (0 restores the device's own stream)."""
        self._check(self._lib.nvmoe_device_set_stream(self._h, ctypes.c_void_p(cuda_stream or None)))

    def synchronize(self, timeout_ns: int = 60_000_000_000) -> None:
        self._check(self._lib.nvmoe_sync(self._h, timeout_ns))

    def probe_mma_rate(self, n_tile: int = 128, k_groups: int = 8192) -> dict:
        """Measured rate of the block-scaled tensor-core instruction of the expert kernels over all SMs."""
        r = capi.MmaProbe()
        self._check(self._lib.nvmoe_probe_mma_rate(self._h, n_tile, k_groups, ctypes.byref(r)))
        return {"n_tile": r.n_tile, "ctas": r.ctas, "mmas_per_cta": r.mmas_per_cta, "elapsed_ms": r.elapsed_ms,
                "cycles_per_mma": r.cycles_per_mma, "tflops": r.tflops, "sm_clock_mhz_nominal": r.sm_clock_mhz_nominal}

    def close(self) -> None:
        if self._h:
            self._lib.nvmoe_device_close(self._h)
            self._h = None


class ResidentBuffer:
    """``VulkanResidentBuffer``: device memory with byte-level read/write and a device address."""

    def __init__(self, device: CudaComputeDevice, byte_capacity: int, _wrap_ptr: int | None = None):
        self.device = device
        handle = ctypes.c_void_p()
        if _wrap_ptr is None:
            device._check(device._lib.nvmoe_buffer_create(device._h, byte_capacity, ctypes.byref(handle)))
        else:
            device._check(device._lib.nvmoe_buffer_wrap(device._h, ctypes.c_void_p(_wrap_ptr), byte_capacity,
                                                        ctypes.byref(handle)))
        self._h = handle
        self.byte_capacity = byte_capacity

    @classmethod
    def wrap(cls, device: CudaComputeDevice, device_ptr: int, byte_capacity: int) -> "ResidentBuffer":
        """A handle over device memory the caller owns (a framework tensor); destroy frees the handle only."""
        return cls(device, byte_capacity, _wrap_ptr=device_ptr)

    def write_bytes(self, data, offset: int = 0) -> None:
        array = np.ascontiguousarray(data) if not isinstance(data, (bytes, bytearray)) else np.frombuffer(data, dtype=np.uint8)
        self.device._check(self.device._lib.nvmoe_buffer_write(self._h, offset, _ptr(array), array.nbytes))

    write_bytes_at = lambda self, offset, data: self.write_bytes(data, offset)  # noqa: E731

    def read_bytes(self, byte_count: int | None = None, offset: int = 0) -> np.ndarray:
        byte_count = self.byte_capacity - offset if byte_count is None else byte_count
        out = np.empty(byte_count, dtype=np.uint8)
        self.device._check(self.device._lib.nvmoe_buffer_read(self._h, offset, _ptr(out), byte_count))
        return out

    def read(self, dtype, count: int | None = None, offset: int = 0) -> np.ndarray:
        itemsize = np.dtype(dtype).itemsize
        nbytes = None if count is None else count * itemsize
        return self.read_bytes(nbytes, offset).view(dtype)

    def fill(self, byte_value: int, offset: int = 0, byte_count: int | None = None) -> None:
        byte_count = self.byte_capacity - offset if byte_count is None else byte_count
        self.device._check(self.device._lib.nvmoe_buffer_fill(self._h, offset, byte_value, byte_count))

    def device_address(self) -> int:
        return int(self.device._lib.nvmoe_buffer_device_address(self._h))

    def mark_dirty(self) -> None:
        """Says that the contents changed behind this handle (through ``device_address``): plans resolve the table again."""
        self.device._check(self.device._lib.nvmoe_buffer_mark_dirty(self._h))

    def destroy(self) -> None:
        if self._h:
            self.device._lib.nvmoe_buffer_destroy(self._h)
            self._h = None


def address_table(device: CudaComputeDevice, resources: list, representations: list | None = None) -> ResidentBuffer:
    """32-byte records {address, byte_count, generation = 1, resident = 1, representation}, the
    way the reference's conformance tests publish them
    (runtime-rs/src/vulkan_compute/mxfp4_tests.rs:1633-1652). representation 0 = compact MXFP4, 1 =
    the same matrix pre-expanded to E4M3 bytes."""
    words = np.zeros(max(len(resources), 1) * 8, dtype=np.uint32)
    for slot, res in enumerate(resources):
        if res is None:
            continue
        if representations is not None:
            words[slot * 8 + 7] = representations[slot]
        address, count = res.device_address(), res.byte_capacity
        words[slot * 8 + 0] = address & 0xFFFFFFFF
        words[slot * 8 + 1] = address >> 32
        words[slot * 8 + 2] = count & 0xFFFFFFFF
        words[slot * 8 + 3] = count >> 32
        words[slot * 8 + 4] = 1
        words[slot * 8 + 6] = 1
    return device.resident_buffer_from(words)


@dataclass
class ExpertBank:
    """Every expert's packaged tensors as separately resident buffers plus the two table pairs."""

    resources: list
    gate_up_addresses: ResidentBuffer
    gate_up_slots: ResidentBuffer
    down_addresses: ResidentBuffer
    down_slots: ResidentBuffer

    def destroy(self) -> None:
        """Frees the tables and every tensor of the bank."""
        for buf in (self.gate_up_addresses, self.gate_up_slots, self.down_addresses, self.down_slots, *self.resources):
            buf.destroy()
        self.resources = []

    @staticmethod
    def upload(device: CudaComputeDevice, w1, s1, w3, s3, w2, s2, present=None, expanded=()) -> "ExpertBank":
        n = len(w1)
        present = set(range(n) if present is None else present)
        per_expert = [[device.resident_buffer_from(t[e]) for t in (w1, s1, w3, s3, w2, s2)] if e in present else None
                      for e in range(n)]
        return ExpertBank.from_resident(device, per_expert, expanded)

    @staticmethod
    def from_resident(device: CudaComputeDevice, per_expert: list, expanded=()) -> "ExpertBank":
        """Tables over tensors that are already resident: `per_expert[e]` is the expert's six buffers
        (w1, w1 scales, w3, w3 scales, w2, w2 scales) or None for an expert this device does not hold.
        The weight records of the experts in `expanded` are tagged representation 1 (pre-expanded E4M3 bytes)."""
        n = len(per_expert)
        gres, dres, greps, dreps = [], [], [], []
        gslots = np.full(n * 4, UNBOUND_PARAMETER_SLOT, dtype=np.uint32)
        dslots = np.full(n * 2, UNBOUND_PARAMETER_SLOT, dtype=np.uint32)
        for e, tensors in enumerate(per_expert):
            if tensors is None:
                continue
            for j, buf in enumerate(tensors[:4]):
                gslots[e * 4 + j] = len(gres)
                gres.append(buf)
                greps.append(1 if (e in expanded and j % 2 == 0) else 0)
            for j, buf in enumerate(tensors[4:]):
                dslots[e * 2 + j] = len(dres)
                dres.append(buf)
                dreps.append(1 if (e in expanded and j % 2 == 0) else 0)
        return ExpertBank(gres + dres, address_table(device, gres, greps), device.resident_buffer_from(gslots),
                          address_table(device, dres, dreps), device.resident_buffer_from(dslots))


def _load_framework_nccl() -> None:
    """The library binds whichever libnccl.so.2 the process already holds, else the system's. PyTorch ships
    its own and cannot start on an older one loaded before it: if PyTorch is installed, let it load first."""
    try:
        import torch  # noqa: F401
    except ImportError:
        pass


class ExpertParallelGroup:
    """This rank's membership of an expert-parallel communicator held by the library (NCCL)."""

    @staticmethod
    def unique_id() -> bytes:
        """Rank 0 makes the id; every rank needs the same 128 bytes to join."""
        _load_framework_nccl()
        buf = ctypes.create_string_buffer(128)
        rc = capi.load().nvmoe_ep_unique_id(buf)
        if rc != 0:
            raise CudaError(rc, capi.load().nvmoe_last_error(None).decode(errors="replace"))
        return buf.raw

    def __init__(self, device: CudaComputeDevice, unique_id: bytes, rank: int, world_size: int):
        assert len(unique_id) == 128
        _load_framework_nccl()
        self.device, self.rank, self.world_size = device, rank, world_size
        handle = ctypes.c_void_p()
        device._check(device._lib.nvmoe_ep_create(device._h, unique_id, rank, world_size, ctypes.byref(handle)))
        self._h = handle

    def layer(self, home: "MoePlan", work: "MoePlan", batch_width, bank: "ExpertBank", hidden, output, owner_table,
              router_weights, router_bias=None, bias=None, telemetry=None, capacity_rows: int = 0) -> None:
        a = capi.EpLayerArgs()
        a.batch_width = batch_width
        a.capacity_rows = capacity_rows
        a.hidden, a.output, a.owner_table = _h(hidden), _h(output), _h(owner_table)
        a.router_weights, a.router_bias, a.bias, a.telemetry = _h(router_weights), _h(router_bias), _h(bias), _h(telemetry)
        a.gate_up_addresses, a.gate_up_slots = _h(bank.gate_up_addresses), _h(bank.gate_up_slots)
        a.down_addresses, a.down_slots = _h(bank.down_addresses), _h(bank.down_slots)
        self.device._check(self.device._lib.nvmoe_ep_layer(self._h, home._h, work._h, ctypes.byref(a)))

    def sync(self, timeout_ns: int = 30_000_000_000) -> None:
        """Bounded wait for the step; aborts the communicator on an asynchronous error or on timeout."""
        self.device._check(self.device._lib.nvmoe_ep_sync(self._h, timeout_ns))

    def destroy(self) -> None:
        if self._h:
            self.device._lib.nvmoe_ep_destroy(self._h)
            self._h = None


def geometry_from_config(cfg: MoeConfig, max_tokens: int) -> capi.Geometry:
    g = capi.Geometry()
    capi.load().nvmoe_geometry_default(ctypes.byref(g), cfg.hidden, cfg.intermediate, cfg.experts, cfg.k)
    g.always_count = cfg.always_count
    g.always_weight = cfg.always_weight
    g.router_kind = cfg.router_kind
    g.activation = cfg.activation
    g.normalize_selected = cfg.normalize_selected
    g.bias_dtype = cfg.bias_dtype
    g.routed_scale = cfg.routed_scale
    g.logit_softcap = cfg.logit_softcap
    g.n_group = cfg.n_group
    g.topk_group = cfg.topk_group
    g.swiglu_limit = cfg.swiglu_limit
    g.swiglu_alpha = cfg.swiglu_alpha
    g.swiglu_up_offset = cfg.swiglu_up_offset
    g.act_block = cfg.act_block
    g.max_tokens = max_tokens
    g.native_fp8_resources = cfg.native_fp8_resources
    return g


def _h(buf):
    return None if buf is None else buf._h


class MoePlan:
    """One MoE layer geometry: create once, run many (the reference's resident kernel dispatches).

    Method names are the reference's operator names; argument order is its binding order.
    """

    def __init__(self, device: CudaComputeDevice, geometry: capi.Geometry):
        self.device = device
        self.geometry = geometry
        handle = ctypes.c_void_p()
        device._check(device._lib.nvmoe_plan_create(device._h, ctypes.byref(geometry), ctypes.byref(handle)))
        self._h = handle
        self.experts_per_token = geometry.routed_k + geometry.always_count
        self.total_experts = geometry.routed_experts + geometry.always_count
        self.frame_words = self.experts_per_token * geometry.intermediate_size // 2 + self.experts_per_token
        self.data_words = self.experts_per_token * geometry.intermediate_size // 2

    @classmethod
    def for_config(cls, device: CudaComputeDevice, cfg: MoeConfig, max_tokens: int) -> "MoePlan":
        return cls(device, geometry_from_config(cfg, max_tokens))

    def _call(self, name, *args):
        self.device._check(getattr(self.device._lib, name)(self._h, *args))

    def set_expert_path(self, path: int) -> None:
        """0 automatic, 1 CUDA-core dequant-GEMV, 2 tcgen05 grouped MMA."""
        self._call("nvmoe_plan_set_expert_path", path)

    def set_wait_limit(self, clock_cycles: int) -> None:
        """SM clock cycles after which a bounded wait inside the tensor-core kernels gives up (0 = default)."""
        self._call("nvmoe_plan_set_wait_limit", clock_cycles)

    def debug_withhold_arrival(self, enabled: bool) -> None:
        """Test aid: CTA 0 of the gate/up kernel leaves out one stage arrival, so that a bounded wait runs out."""
        self._call("nvmoe_plan_debug_withhold_arrival", int(enabled))

    def set_profiling(self, enabled: bool) -> None:
        self._call("nvmoe_plan_set_profiling", int(enabled))

    def status(self) -> int:
        bits = ctypes.c_uint32()
        self._call("nvmoe_plan_status", ctypes.byref(bits))
        return bits.value

    def telemetry_words(self) -> int:
        r = self.total_experts
        return r + r * (r - 1) // 2

    # -- operators, in chain order ---------------------------------------------------------
    def linear(self, batch_width, hidden, logits, router_weights, router_bias=None):
        self._call("nvmoe_router_linear", batch_width, _h(hidden), _h(logits), _h(router_weights), _h(router_bias))

    def moe_route(self, batch_width, logits, routes, bias=None, telemetry=None):
        self._call("nvmoe_route", batch_width, _h(logits), _h(routes), _h(bias), _h(telemetry))

    def parameter_table_resource_preselection(self, batch_width, token_ids, resource_routes, table, vocab_size,
                                              table_word_stride=1, telemetry=None):
        self._call("nvmoe_resource_preselect_table", batch_width, _h(token_ids), _h(resource_routes), _h(table), vocab_size,
                   table_word_stride, _h(telemetry))

    def moe_route_preselected(self, batch_width, logits, resource_routes, routes):
        self._call("nvmoe_route_preselected", batch_width, _h(logits), _h(resource_routes), _h(routes))

    def rms_norm(self, rows, element_count, input, output, weight, eps, weight_offset=0.0):
        self._call("nvmoe_rms_norm", rows, element_count, _h(input), _h(output), _h(weight), eps, weight_offset)

    def silu_multiply(self, rows, element_count, gate, up, output, limit=0.0):
        """`bounded_silu_multiply` with limit > 0, `silu_multiply` with limit 0."""
        self._call("nvmoe_silu_multiply", rows, element_count, _h(gate), _h(up), _h(output), limit)

    def residual_add(self, rows, element_count, a, b, output):
        self._call("nvmoe_residual_add", rows, element_count, _h(a), _h(b), _h(output))

    def dense_linear(self, batch_width, input, output, weights, scales, rows, cols):
        self._call("nvmoe_dense_linear", batch_width, _h(input), _h(output), _h(weights), _h(scales), rows, cols)

    def moe_route_compact(self, batch_width, routes, intermediates, control, slots=None):
        self._call("nvmoe_route_compact", batch_width, _h(routes), _h(intermediates), _h(slots), _h(control))

    def moe_route_compact_static(self, batch_width, routes, intermediates, control, slots=None):
        """moe_route_compact with the sort scratch in the library's fixed device array: no device allocation."""
        self._call("nvmoe_route_compact_static", batch_width, _h(routes), _h(intermediates), _h(slots), _h(control))

    def moe_route_count(self, batch_width, routes, control, slots=None):
        self._call("nvmoe_route_count", batch_width, _h(routes), _h(slots), _h(control))

    def quantize_fp8_e4m3(self, rows, columns, input, quantized, scales):
        self._call("nvmoe_quantize_fp8", rows, columns, _h(input), _h(quantized), _h(scales))

    def independent_sparse_moe_gate_up(self, batch_width, hidden, routes, intermediates, addresses, slots, control):
        self._call("nvmoe_gate_up", batch_width, _h(hidden), _h(routes), _h(intermediates), _h(addresses), _h(slots),
                   _h(control))

    def independent_sparse_moe_gate_up_prequant(self, batch_width, q_hidden, scales, routes, intermediates,
                                                addresses, slots, control):
        self._call("nvmoe_gate_up_prequant", batch_width, _h(q_hidden), _h(scales), _h(routes), _h(intermediates),
                   _h(addresses), _h(slots), _h(control))

    def independent_sparse_moe_down(self, batch_width, intermediates, routes, outputs, addresses, slots, control):
        self._call("nvmoe_down", batch_width, _h(intermediates), _h(routes), _h(outputs), _h(addresses), _h(slots),
                   _h(control))

    def independent_sparse_moe_down_partial(self, batch_width, intermediates, routes, partial_outputs, addresses, slots, control):
        """The tensor-parallel form of the down projection: raw f32 sums over this participant's column range."""
        self._call("nvmoe_down_partial", batch_width, _h(intermediates), _h(routes), _h(partial_outputs), _h(addresses),
                   _h(slots), _h(control))

    def sum_f32_scale_packed_bf16(self, partials, scales, output, element_count, participant_count, lane_count,
                                  elements_per_scale, scale_bit_offset=16):
        self._call("nvmoe_sum_f32_scale_packed_bf16", _h(partials), _h(scales), _h(output), element_count, participant_count,
                   lane_count, elements_per_scale, scale_bit_offset)

    def moe_reduce(self, batch_width, expert_outputs, output):
        self._call("nvmoe_reduce", batch_width, _h(expert_outputs), _h(output))

    # -- expert-parallel exchange ------------------------------------------------------------
    def ep_pack(self, batch_width, hidden, routes, owner_table, world_size, rank, send_rows, send_routes, send_index,
                dest_counts, segment_rows=0):
        self._call("nvmoe_ep_pack", batch_width, _h(hidden), _h(routes), _h(owner_table), world_size, rank,
                   _h(send_rows), _h(send_routes), _h(send_index), _h(dest_counts), segment_rows)

    def ep_unpack(self, batch_width, returned_rows, send_index, expert_outputs):
        self._call("nvmoe_ep_unpack", batch_width, _h(returned_rows), _h(send_index), _h(expert_outputs))

    # -- a node chain, entry point by entry point ------------------------------------------------
    # argument order of every entry point a dispatch list may name: (binding names..., scalar names...)
    _ENTRY_ARGUMENTS = {
        "nvmoe_router_linear": (("hidden", "logits", "router_weights", "router_bias"), ()),
        "nvmoe_route": (("logits", "routes", "bias", "telemetry"), ()),
        "nvmoe_resource_preselect_table": (("token_ids", "resource_routes", "table"), ("vocab_size", "table_word_stride", "telemetry")),
        "nvmoe_route_preselected": (("logits", "resource_routes", "routes"), ()),
        "nvmoe_route_compact": (("routes", "intermediates", "slots", "control"), ()),
        "nvmoe_gate_up": (("hidden", "routes", "intermediates", "addresses", "slots", "control"), ()),
        "nvmoe_route_count": (("routes", "slots", "control"), ()),
        "nvmoe_down": (("intermediates", "routes", "outputs", "addresses", "slots", "control"), ()),
        "nvmoe_reduce": (("expert_outputs", "output"), ()),
        "nvmoe_dense_linear": (("input", "output", "weights", "scales"), ("rows", "cols")),
        "nvmoe_silu_multiply": (("#element_count", "gate", "up", "output"), ("limit",)),
        "nvmoe_residual_add": (("#element_count", "a", "b", "output"), ()),
    }

    def run_dispatch(self, dispatch, batch_width: int, buffers: dict, expert_start: int = 0, expert_count: int = 0) -> None:
        """Runs the dispatch list of ``node_chain.plan_from_nodes`` one entry point per node, the way a runtime
        that walks the component's kernel steps would: ``buffers`` maps every signal and parameter id the list
        names (plus ``<node>.address_table`` / ``<node>.parameter_slots`` of the two expert nodes) to a resident
        buffer. The 7-word control blocks of the scheduler stages are created here and written as the reference
        host writes them ({batch_width, expert_start, expert_count, 0, 0, 0, 0})."""
        control_words = np.array([batch_width, expert_start, expert_count, 0, 0, 0, 0], dtype=np.uint32)
        for step in dispatch.steps:
            names, scalar_names = self._ENTRY_ARGUMENTS[step.entry]
            bound = dict(step.bindings)
            args = [batch_width]
            for name in names:
                if name.startswith("#"):
                    args.append(step.scalars[name[1:]])
                    continue
                key = bound.get(name)
                if key is not None and key.endswith(".control") and key not in buffers:
                    buffers[key] = self.device.resident_buffer_from(control_words)
                elif key is not None and key.endswith(".control") and step.entry in ("nvmoe_route_compact", "nvmoe_route_count"):
                    buffers[key].write_bytes(control_words)
                args.append(_h(buffers.get(key)) if key is not None else None)
            for name in scalar_names:
                args.append(_h(buffers.get(dict(step.bindings).get(name))) if name == "telemetry" else step.scalars[name])
            self._call(step.entry, *args)

    def launches(self) -> int:
        """Kernels this plan has launched since it was created."""
        return int(self.device._lib.nvmoe_plan_launch_count(self._h))

    # -- the whole chain -------------------------------------------------------------------
    def _layer_args(self, batch_width, bank: ExpertBank, hidden=None, output=None, router_weights=None,
                    router_bias=None, logits=None, bias=None, routes_out=None, telemetry=None, expert_start=0,
                    expert_count=0, routes_in=None, expert_outputs=None) -> capi.LayerArgs:
        a = capi.LayerArgs()
        a.batch_width, a.expert_start, a.expert_count = batch_width, expert_start, expert_count
        a.hidden, a.output = _h(hidden), _h(output)
        a.router_weights, a.router_bias, a.logits, a.bias = _h(router_weights), _h(router_bias), _h(logits), _h(bias)
        a.gate_up_addresses, a.gate_up_slots = _h(bank.gate_up_addresses), _h(bank.gate_up_slots)
        a.down_addresses, a.down_slots = _h(bank.down_addresses), _h(bank.down_slots)
        a.routes_out, a.telemetry = _h(routes_out), _h(telemetry)
        a.routes_in, a.expert_outputs = _h(routes_in), _h(expert_outputs)
        return a

    def layer(self, batch_width, bank: ExpertBank, hidden, output, **kw):
        args = self._layer_args(batch_width, bank, hidden=hidden, output=output, **kw)
        self._call("nvmoe_layer", ctypes.byref(args))

    def layer_host(self, batch_width, bank: ExpertBank, hidden_host: np.ndarray, output_host: np.ndarray, **kw):
        """Host buffers in, host buffers out: the copies are inside the call."""
        assert hidden_host.flags["C_CONTIGUOUS"] and output_host.flags["C_CONTIGUOUS"]
        args = self._layer_args(batch_width, bank, **kw)
        self._call("nvmoe_layer_host", ctypes.byref(args), _ptr(hidden_host), _ptr(output_host))

    def last_report(self) -> dict:
        r = capi.WorkReport()
        self._call("nvmoe_plan_last_report", ctypes.byref(r))
        return {
            "total_ms": r.total_ms,
            "stage_ms": dict(zip(capi.STAGE_NAMES, list(r.stage_ms))),
            "gate_up_kernel_ms": r.gate_up_kernel_ms,
            "down_kernel_ms": r.down_kernel_ms,
            "tensor_path": bool(r.tensor_path),
            "batch_width": r.batch_width,
            "routes": r.routes,
            "distinct_experts": r.distinct_experts,
            "kernel_launches": r.kernel_launches,
            "weight_bytes_touched": r.weight_bytes_touched,
        }

    def destroy(self) -> None:
        if self._h:
            self.device._lib.nvmoe_plan_destroy(self._h)
            self._h = None
