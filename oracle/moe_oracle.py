"""numpy front end of the CPU checker in ``moe_oracle.c``.  TEST INFRASTRUCTURE ONLY.

Imported by the tests, by the smoke check and by the benchmark's CPU-baseline leg.  The product
package never imports this module and has no CPU fallback.

Every function takes and returns numpy arrays in the buffer layouts of the reference shaders
(packed bf16 words, route words, intermediate frames, 7-word control blocks, 32-byte address
records).  Address tables built by :func:`address_table` hold host pointers to the numpy arrays
passed in; the caller must keep those arrays alive while the table is in use.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from dataclasses import dataclass
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_LIB_PATH = _HERE / "libmoe_oracle.so"

UNBOUND_SLOT = 0xFFFFFFFF


def build(force: bool = False) -> Path:
    """Compile the checker with the Makefile beside it (gcc only, a second or two)."""
    sources = [_HERE / "moe_oracle.c", _HERE / "moe_oracle.h", _HERE.parent / "include" / "nvmoe_math.h"]
    stale = not _LIB_PATH.exists() or any(
        s.stat().st_mtime > _LIB_PATH.stat().st_mtime for s in sources if s.exists()
    )
    if force or stale:
        subprocess.run(["make", "-C", str(_HERE), "-B", "libmoe_oracle.so"], check=True, capture_output=True)
    return _LIB_PATH


class _Router(ctypes.Structure):
    _fields_ = [
        ("routed_experts", ctypes.c_uint32),
        ("routed_k", ctypes.c_uint32),
        ("always_count", ctypes.c_uint32),
        ("always_weight", ctypes.c_float),
        ("kind", ctypes.c_uint32),
        ("activation", ctypes.c_uint32),
        ("normalize_selected", ctypes.c_uint32),
        ("bias_dtype", ctypes.c_uint32),
        ("routed_scale", ctypes.c_float),
        ("logit_softcap", ctypes.c_float),
        ("n_group", ctypes.c_uint32),
        ("topk_group", ctypes.c_uint32),
    ]


class _Expert(ctypes.Structure):
    _fields_ = [
        ("hidden_size", ctypes.c_uint32),
        ("intermediate_size", ctypes.c_uint32),
        ("num_experts", ctypes.c_uint32),
        ("experts_per_token", ctypes.c_uint32),
        ("tile_rows", ctypes.c_uint32),
        ("swiglu_limit", ctypes.c_float),
        ("swiglu_alpha", ctypes.c_float),
        ("swiglu_up_offset", ctypes.c_float),
        ("act_block", ctypes.c_uint32),
        ("tier", ctypes.c_uint32),
        ("native_fp8_start", ctypes.c_uint32),
    ]


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(str(_LIB_PATH))
        f32, u32 = ctypes.c_float, ctypes.c_uint32
        for name, res, args in [
            ("oracle_e2m1_to_e4m3", u32, [u32]),
            ("oracle_e2m1_value", f32, [u32]),
            ("oracle_e4m3_value", f32, [u32]),
            ("oracle_f32_to_e4m3", u32, [f32]),
            ("oracle_e8m0_value", f32, [u32]),
            ("oracle_rounded_fp8_scale", f32, [f32]),
            ("oracle_f32_to_bf16", u32, [f32]),
            ("oracle_expf", f32, [f32]),
            ("oracle_logf", f32, [f32]),
            ("oracle_tanhf", f32, [f32]),
            ("oracle_max_threads", ctypes.c_int, []),
            ("oracle_set_threads", ctypes.c_int, [ctypes.c_int]),
        ]:
            fn = getattr(_lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib.oracle_route.restype = ctypes.c_int
    return _lib


def _p(a):
    if a is None:
        return None
    return a.ctypes.data_as(ctypes.c_void_p)


def _c(a, dtype):
    a = np.ascontiguousarray(a, dtype=dtype)
    return a


# --------------------------------------------------------------------------------------------
# bf16 helpers (numpy has no bf16: values travel as uint16 bit patterns)


def f32_to_bf16(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even on the bit pattern, as every reference shader does."""
    bits = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    lsb = (bits >> 16) & 1
    return (((bits + 0x7FFF + lsb) >> 16) & 0xFFFF).astype(np.uint16)


def bf16_to_f32(h: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(h, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


# --------------------------------------------------------------------------------------------


@dataclass
class RouterParams:
    routed_experts: int
    routed_k: int
    always_count: int = 0
    always_weight: float = 1.0
    kind: int = 0
    activation: int = 0
    normalize_selected: int = 0
    bias_dtype: int = 0
    routed_scale: float = 1.0
    logit_softcap: float = 0.0
    n_group: int = 0
    topk_group: int = 0

    @property
    def total_k(self) -> int:
        return self.routed_k + (self.always_count if self.kind in (0, 3) else 0)

    @property
    def total_resources(self) -> int:
        return self.routed_experts + (self.always_count if self.kind in (0, 3) else 0)

    def telemetry_words(self) -> int:
        r = self.total_resources
        return r + r * (r - 1) // 2

    def c(self) -> _Router:
        return _Router(
            self.routed_experts, self.routed_k, self.always_count if self.kind in (0, 3) else 0,
            self.always_weight, self.kind, self.activation, self.normalize_selected,
            self.bias_dtype, self.routed_scale, self.logit_softcap, self.n_group, self.topk_group,
        )


@dataclass
class ExpertParams:
    hidden_size: int
    intermediate_size: int
    num_experts: int
    experts_per_token: int
    tile_rows: int = 32
    swiglu_limit: float = 0.0
    swiglu_alpha: float = 1.0
    swiglu_up_offset: float = 0.0
    act_block: int = 128
    tier: int = 1
    native_fp8_start: int = 0  # resources from here on hold native FP8 weights (0 = none)

    @property
    def frame_words(self) -> int:
        return self.experts_per_token * self.intermediate_size // 2 + self.experts_per_token

    @property
    def data_words(self) -> int:
        return self.experts_per_token * self.intermediate_size // 2

    def c(self) -> _Expert:
        return _Expert(
            self.hidden_size, self.intermediate_size, self.num_experts, self.experts_per_token,
            self.tile_rows, self.swiglu_limit, self.swiglu_alpha, self.swiglu_up_offset,
            self.act_block, self.tier, self.native_fp8_start,
        )


def linear_bf16(x_bf16: np.ndarray, w_bf16: np.ndarray, bias_bf16: np.ndarray | None = None) -> np.ndarray:
    """[T,H] x [E,H]^T (+ bias) -> packed bf16 logit words [T, ceil(E/2)]."""
    x = _c(x_bf16, np.uint16)
    w = _c(w_bf16, np.uint16)
    b = None if bias_bf16 is None else _c(bias_bf16, np.uint16)
    tokens, hidden = x.shape
    outputs = w.shape[0]
    out = np.zeros((tokens, (outputs + 1) // 2), dtype=np.uint32)
    lib().oracle_linear_bf16(_p(x), _p(w), _p(b), ctypes.c_uint32(tokens), ctypes.c_uint32(hidden),
                             ctypes.c_uint32(outputs), _p(out))
    return out


def route(p: RouterParams, logit_words: np.ndarray, bias: np.ndarray | None = None,
          telemetry: np.ndarray | None = None):
    """Returns (routes [T, K_total] uint32, tokens_without_candidates)."""
    assert p.total_k <= 64
    lw = _c(logit_words, np.uint32)
    tokens = lw.shape[0]
    assert lw.shape[1] == (p.routed_experts + 1) // 2
    if p.bias_dtype == 1:
        bias = _c(bias, np.float32)
    elif p.bias_dtype == 2:
        bias = _c(bias, np.uint16)
    else:
        bias = None
    routes = np.zeros((tokens, p.total_k), dtype=np.uint32)
    if telemetry is not None:
        assert telemetry.dtype == np.uint32 and telemetry.size >= p.telemetry_words()
    cp = p.c()
    bad = lib().oracle_route(ctypes.byref(cp), _p(lw), _p(bias), ctypes.c_uint32(tokens), _p(routes),
                             _p(telemetry))
    return routes, bad


def route_compact(routes: np.ndarray, intermediates: np.ndarray, control: np.ndarray,
                  intermediate_size: int, experts_per_token: int, tiles_per_route: int,
                  slots: np.ndarray | None = None, params_per_resource: int = 4,
                  quadratic: bool = False) -> None:
    """Runs the route scheduler in place on ``intermediates`` (schedule words) and ``control``."""
    r = _c(routes, np.uint32)
    assert intermediates.dtype == np.uint32 and control.dtype == np.uint32 and control.size == 7
    if quadratic:
        assert control[2] == 0
        lib().oracle_route_compact_quadratic(_p(r), _p(intermediates), _p(control),
                                             ctypes.c_uint32(intermediate_size),
                                             ctypes.c_uint32(experts_per_token),
                                             ctypes.c_uint32(tiles_per_route))
        return
    s = None if slots is None else _c(slots, np.uint32)
    lib().oracle_route_compact(_p(r), _p(intermediates), _p(s),
                               ctypes.c_uint32(0 if s is None else s.size),
                               ctypes.c_uint32(params_per_resource), _p(control),
                               ctypes.c_uint32(intermediate_size), ctypes.c_uint32(experts_per_token),
                               ctypes.c_uint32(tiles_per_route))


def route_count(routes: np.ndarray, control: np.ndarray, experts_per_token: int,
                tiles_per_route: int, slots: np.ndarray | None = None,
                params_per_resource: int = 2) -> None:
    r = _c(routes, np.uint32)
    s = None if slots is None else _c(slots, np.uint32)
    lib().oracle_route_count(_p(r), _p(s), ctypes.c_uint32(0 if s is None else s.size),
                             ctypes.c_uint32(params_per_resource), _p(control),
                             ctypes.c_uint32(experts_per_token), ctypes.c_uint32(tiles_per_route))


def quantize_fp8(x_bf16: np.ndarray, block: int):
    x = _c(x_bf16, np.uint16)
    rows, cols = x.shape
    q = np.zeros((rows, cols), dtype=np.uint8)
    scales = np.zeros((rows, cols // block), dtype=np.float32)
    lib().oracle_quantize_fp8(_p(x), ctypes.c_uint32(rows), ctypes.c_uint32(cols),
                              ctypes.c_uint32(block), _p(q), _p(scales))
    return q, scales


def address_table(resources: list[np.ndarray | None], representations: list | None = None) -> np.ndarray:
    """32-byte records {address, byte_count, generation=1, resident=1, representation} with
    host pointers, as the reference test helper builds them
    (runtime-rs/src/vulkan_compute/mxfp4_tests.rs:1633-1652). ``None`` leaves a zero record."""
    words = np.zeros(len(resources) * 8, dtype=np.uint32)
    for slot, res in enumerate(resources):
        if representations is not None:
            words[slot * 8 + 7] = representations[slot]
        if res is None:
            continue
        assert res.flags["C_CONTIGUOUS"]
        address = res.ctypes.data
        words[slot * 8] = address & 0xFFFFFFFF
        words[slot * 8 + 1] = address >> 32
        words[slot * 8 + 2] = res.nbytes & 0xFFFFFFFF
        words[slot * 8 + 3] = res.nbytes >> 32
        words[slot * 8 + 4] = 1
        words[slot * 8 + 6] = 1
    return words


def gate_up(p: ExpertParams, hidden_bf16: np.ndarray, routes: np.ndarray, intermediates: np.ndarray,
            addresses: np.ndarray, slots: np.ndarray, control: np.ndarray) -> None:
    h = _c(hidden_bf16, np.uint16)
    r = _c(routes, np.uint32)
    a = _c(addresses, np.uint32)
    s = _c(slots, np.uint32)
    c = _c(control, np.uint32)
    assert intermediates.dtype == np.uint32 and intermediates.flags["C_CONTIGUOUS"]
    cp = p.c()
    lib().oracle_gate_up(ctypes.byref(cp), _p(h), _p(r), _p(intermediates), _p(a),
                         ctypes.c_uint32(a.size), _p(s), ctypes.c_uint32(s.size), _p(c))


def gate_up_prequant(p: ExpertParams, q_hidden: np.ndarray, hidden_scales: np.ndarray,
                     routes: np.ndarray, intermediates: np.ndarray, addresses: np.ndarray,
                     slots: np.ndarray, control: np.ndarray) -> None:
    q = _c(q_hidden, np.uint8)
    hs = _c(hidden_scales, np.float32)
    r = _c(routes, np.uint32)
    a = _c(addresses, np.uint32)
    s = _c(slots, np.uint32)
    c = _c(control, np.uint32)
    assert intermediates.dtype == np.uint32 and intermediates.flags["C_CONTIGUOUS"]
    cp = p.c()
    lib().oracle_gate_up_prequant(ctypes.byref(cp), _p(q), _p(hs), _p(r), _p(intermediates), _p(a),
                                  ctypes.c_uint32(a.size), _p(s), ctypes.c_uint32(s.size), _p(c))


def down(p: ExpertParams, intermediates: np.ndarray, routes: np.ndarray, outputs: np.ndarray,
         addresses: np.ndarray, slots: np.ndarray, control: np.ndarray) -> None:
    i = _c(intermediates, np.uint32)
    r = _c(routes, np.uint32)
    a = _c(addresses, np.uint32)
    s = _c(slots, np.uint32)
    c = _c(control, np.uint32)
    assert outputs.dtype == np.uint16 and outputs.flags["C_CONTIGUOUS"]
    cp = p.c()
    lib().oracle_down(ctypes.byref(cp), _p(i), _p(r), _p(outputs), _p(a), ctypes.c_uint32(a.size),
                      _p(s), ctypes.c_uint32(s.size), _p(c))


def reduce(expert_outputs: np.ndarray, tokens: int, experts_per_token: int, hidden: int,
           routed_scale: float = 1.0) -> np.ndarray:
    e = _c(expert_outputs, np.uint16)
    out = np.zeros((tokens, hidden), dtype=np.uint16)
    lib().oracle_reduce(_p(e), _p(out), ctypes.c_uint32(tokens), ctypes.c_uint32(experts_per_token),
                        ctypes.c_uint32(hidden), ctypes.c_float(routed_scale))
    return out


def sum_f32_scale_packed_bf16(partials: np.ndarray, scales: np.ndarray, element_count: int,
                              participant_count: int, lane_count: int, elements_per_scale: int,
                              scale_bit_offset: int) -> np.ndarray:
    pa = _c(partials, np.float32)
    sc = _c(scales, np.uint32)
    out = np.zeros(lane_count * element_count // 2, dtype=np.uint32)
    lib().oracle_sum_f32_scale_packed_bf16(_p(pa), _p(sc), _p(out), ctypes.c_uint32(element_count),
                                           ctypes.c_uint32(participant_count),
                                           ctypes.c_uint32(lane_count),
                                           ctypes.c_uint32(elements_per_scale),
                                           ctypes.c_uint32(scale_bit_offset))
    return out


def resource_preselect_table(token_ids: np.ndarray, table: np.ndarray, routed: int, k: int, always: int = 0,
                             telemetry: np.ndarray | None = None):
    """Returns (selections [T, k + always] uint32, invalid token count). `table` is [vocab, k] int32 or int64."""
    assert table.dtype in (np.int32, np.int64) and table.ndim == 2 and table.shape[1] == k
    ids = _c(token_ids, np.uint32)
    words = np.ascontiguousarray(table).view(np.uint32)
    stride = table.dtype.itemsize // 4
    out = np.zeros((ids.size, k + always), dtype=np.uint32)
    lib().oracle_resource_preselect_table.restype = ctypes.c_int
    bad = lib().oracle_resource_preselect_table(_p(ids), _p(words), ctypes.c_uint32(stride), ctypes.c_uint32(table.shape[0]),
                                                ctypes.c_uint32(routed), ctypes.c_uint32(k), ctypes.c_uint32(always),
                                                ctypes.c_uint32(ids.size), _p(out), _p(telemetry))
    return out, bad


def route_preselected(p: RouterParams, logit_words: np.ndarray, selections: np.ndarray) -> np.ndarray:
    lw = _c(logit_words, np.uint32)
    sel = _c(selections, np.uint32)
    routes = np.zeros_like(sel)
    cp = p.c()
    lib().oracle_route_preselected(ctypes.byref(cp), _p(lw), _p(sel), ctypes.c_uint32(lw.shape[0]), _p(routes))
    return routes


def rms_norm(x_bf16: np.ndarray, weight_bf16: np.ndarray, eps: float, weight_offset: float = 0.0) -> np.ndarray:
    x = _c(x_bf16, np.uint16)
    w = _c(weight_bf16, np.uint16)
    out = np.zeros_like(x)
    lib().oracle_rms_norm(_p(x), _p(w), _p(out), ctypes.c_uint32(x.shape[0]), ctypes.c_uint32(x.shape[1]),
                          ctypes.c_float(eps), ctypes.c_float(weight_offset))
    return out


def silu_multiply(gate_bf16: np.ndarray, up_bf16: np.ndarray, limit: float = 0.0) -> np.ndarray:
    g, u = _c(gate_bf16, np.uint16), _c(up_bf16, np.uint16)
    out = np.zeros_like(g)
    lib().oracle_silu_multiply(_p(g), _p(u), _p(out), ctypes.c_uint64(g.size), ctypes.c_float(limit))
    return out


def add_bf16(a_bf16: np.ndarray, b_bf16: np.ndarray) -> np.ndarray:
    a, b = _c(a_bf16, np.uint16), _c(b_bf16, np.uint16)
    out = np.zeros_like(a)
    lib().oracle_add_bf16(_p(a), _p(b), _p(out), ctypes.c_uint64(a.size))
    return out


def dense_linear_mxfp4(x_bf16: np.ndarray, weight: np.ndarray, scales: np.ndarray, act_block: int, tier: int = 1) -> np.ndarray:
    """A dense linear over packaged MXFP4 weights [rows, cols/2] + [rows, cols/32] with the expert kernels'
    arithmetic (activations quantised per `act_block`, f32 or f64 accumulation, one bf16 rounding): the down
    projection of a single always-selected resource with route weight 1."""
    x = _c(x_bf16, np.uint16)
    tokens, cols = x.shape
    rows = weight.shape[0]
    ep = ExpertParams(hidden_size=rows, intermediate_size=cols, num_experts=1, experts_per_token=1, act_block=act_block, tier=tier)
    frames = np.zeros((tokens, ep.frame_words), dtype=np.uint32)
    frames[:, : cols // 2] = x.view(np.uint32)
    frames[:, cols // 2] = np.arange(tokens, dtype=np.uint32)
    routes = np.full((tokens, 1), 0x3F80 << 16, dtype=np.uint32)
    w, sc = _c(weight, np.uint8), _c(scales, np.uint8)
    out = np.zeros((tokens, 1, rows), dtype=np.uint16)
    control = np.array([tokens, 0, 0, 0, 0, 0, 0], dtype=np.uint32)
    down(ep, frames, routes, out, address_table([w, sc]), np.array([0, 1], dtype=np.uint32), control)
    return out.reshape(tokens, rows)


def dequant_mxfp4(packed: np.ndarray, scales: np.ndarray) -> np.ndarray:
    pk = _c(packed, np.uint8)
    sc = _c(scales, np.uint8)
    rows, half = pk.shape
    out = np.zeros((rows, half * 2), dtype=np.float32)
    lib().oracle_dequant_mxfp4(_p(pk), _p(sc), ctypes.c_uint32(rows), ctypes.c_uint32(half * 2), _p(out))
    return out


@dataclass
class ExpertWeights:
    """Packaged MXFP4 tensors of every expert: w1/w3 [I, H/2] + [I, H/32], w2 [H, I/2] + [H, I/32]."""

    w1: list
    s1: list
    w3: list
    s3: list
    w2: list
    s2: list
    expanded: frozenset = frozenset()  # experts whose weight records say "pre-expanded FP8" (representation 1)

    def gate_up_tables(self, present=None):
        """(address words, slot words, keepalive) with P = 4 per expert."""
        n = len(self.w1)
        present = range(n) if present is None else present
        resources, reps, slots = [], [], np.full(n * 4, UNBOUND_SLOT, dtype=np.uint32)
        for e in present:
            for j, arr in enumerate((self.w1[e], self.s1[e], self.w3[e], self.s3[e])):
                slots[e * 4 + j] = len(resources)
                resources.append(arr)
                reps.append(1 if (e in self.expanded and j % 2 == 0) else 0)
        return address_table(resources, reps), slots

    def down_tables(self, present=None):
        n = len(self.w2)
        present = range(n) if present is None else present
        resources, reps, slots = [], [], np.full(n * 2, UNBOUND_SLOT, dtype=np.uint32)
        for e in present:
            for j, arr in enumerate((self.w2[e], self.s2[e])):
                slots[e * 2 + j] = len(resources)
                resources.append(arr)
                reps.append(1 if (e in self.expanded and j % 2 == 0) else 0)
        return address_table(resources, reps), slots


def moe_layer(rp: RouterParams, ep: ExpertParams, hidden_bf16: np.ndarray, logit_words: np.ndarray,
              bias, weights: ExpertWeights, expert_start: int = 0, expert_count: int = 0,
              down_tile_rows: int = 64, reduce_scale: float = 1.0):
    """The node chain of nerve/circuit_lowering_sparse_experts.py:80-172 on the CPU:
    moe_route -> compact -> gate_up -> count -> down -> moe_reduce.
    Returns (output bf16 [T,H], routes, expert_outputs, intermediates frames)."""
    tokens = hidden_bf16.shape[0]
    K, I, H = ep.experts_per_token, ep.intermediate_size, ep.hidden_size
    routes, bad = route(rp, logit_words, bias)
    assert bad == 0
    inter = np.zeros((tokens, ep.frame_words), dtype=np.uint32)
    gaddr, gslots = weights.gate_up_tables()
    daddr, dslots = weights.down_tables()
    control = np.array([tokens, expert_start, expert_count, 0, 0, 0, 0], dtype=np.uint32)
    route_compact(routes, inter, control, I, K, -(-I // ep.tile_rows), slots=gslots)
    gate_up(ep, hidden_bf16, routes, inter, gaddr, gslots, control)
    dcontrol = np.array([tokens, expert_start, expert_count, 0, 0, 0, 0], dtype=np.uint32)
    route_count(routes, dcontrol, K, -(-H // down_tile_rows), slots=dslots)
    outputs = np.zeros((tokens, K, H), dtype=np.uint16)
    down(ep, inter, routes, outputs, daddr, dslots, dcontrol)
    out = reduce(outputs, tokens, K, H, reduce_scale)
    return out, routes, outputs, inter


def router_params_from(cfg) -> RouterParams:
    """RouterParams of a ``nerve_b200.synthetic.MoeConfig`` (duck-typed: the checker imports no product code)."""
    return RouterParams(
        routed_experts=cfg.experts, routed_k=cfg.k, always_count=cfg.always_count,
        always_weight=cfg.always_weight, kind=cfg.router_kind, activation=cfg.activation,
        normalize_selected=cfg.normalize_selected, bias_dtype=cfg.bias_dtype, routed_scale=cfg.routed_scale,
        logit_softcap=cfg.logit_softcap, n_group=cfg.n_group, topk_group=cfg.topk_group)


def expert_params_from(cfg, tier: int = 1) -> ExpertParams:
    return ExpertParams(
        hidden_size=cfg.hidden, intermediate_size=cfg.intermediate, num_experts=cfg.total_experts,
        experts_per_token=cfg.total_k, tile_rows=32, swiglu_limit=cfg.swiglu_limit,
        swiglu_alpha=cfg.swiglu_alpha, swiglu_up_offset=cfg.swiglu_up_offset, act_block=cfg.act_block, tier=tier,
        native_fp8_start=(cfg.total_experts - cfg.native_fp8_resources) if getattr(cfg, "native_fp8_resources", 0) else 0)
