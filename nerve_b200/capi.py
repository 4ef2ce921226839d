"""ctypes binding of ``libnerve_cuda_moe.so`` — the declarations of ``include/nerve_cuda_moe.h``.

Loading fails loudly when the library has not been built: there is no CPU fallback.
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, c_char_p, c_float, c_int, c_size_t, c_uint32, c_uint64, c_void_p
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libnerve_cuda_moe.so"

NVMOE_OK = 0
ERR_INVALID_ARGUMENT, ERR_CUDA, ERR_TIMEOUT, ERR_OUT_OF_MEMORY, ERR_UNSUPPORTED, ERR_COLLECTIVE, ERR_DEVICE_STATUS = (
    -1, -2, -3, -4, -5, -6, -7)
STATUS_ROUTE_NONFINITE, STATUS_ROUTE_OUT_OF_RANGE, STATUS_EXPERT_NOT_RESIDENT, STATUS_WAIT_EXPIRED = 1, 2, 4, 8
STATUS_EXCHANGE_OVERFLOW = 16
STAGE_NAMES = ("linear", "route", "schedule", "quantize_hidden", "gate_up", "quantize_intermediate", "down", "reduce")


class Geometry(ctypes.Structure):
    _fields_ = [
        ("hidden_size", c_uint32), ("intermediate_size", c_uint32), ("routed_experts", c_uint32),
        ("routed_k", c_uint32), ("always_count", c_uint32), ("always_weight", c_float),
        ("router_kind", c_uint32), ("activation", c_uint32), ("normalize_selected", c_uint32),
        ("bias_dtype", c_uint32), ("routed_scale", c_float), ("logit_softcap", c_float),
        ("n_group", c_uint32), ("topk_group", c_uint32), ("swiglu_limit", c_float),
        ("swiglu_alpha", c_float), ("swiglu_up_offset", c_float), ("act_block", c_uint32),
        ("gate_tile_rows", c_uint32), ("down_tile_rows", c_uint32), ("reduce_scale", c_float),
        ("max_tokens", c_uint32), ("native_fp8_resources", c_uint32),
    ]


class LayerArgs(ctypes.Structure):
    _fields_ = [
        ("batch_width", c_uint32), ("expert_start", c_uint32), ("expert_count", c_uint32),
        ("hidden", c_void_p), ("router_weights", c_void_p), ("router_bias", c_void_p), ("logits", c_void_p),
        ("bias", c_void_p), ("gate_up_addresses", c_void_p), ("gate_up_slots", c_void_p),
        ("down_addresses", c_void_p), ("down_slots", c_void_p), ("output", c_void_p),
        ("routes_out", c_void_p), ("telemetry", c_void_p), ("routes_in", c_void_p), ("expert_outputs", c_void_p),
    ]


class EpLayerArgs(ctypes.Structure):
    _fields_ = [
        ("batch_width", c_uint32), ("hidden", c_void_p), ("router_weights", c_void_p), ("router_bias", c_void_p),
        ("bias", c_void_p), ("owner_table", c_void_p), ("gate_up_addresses", c_void_p), ("gate_up_slots", c_void_p),
        ("down_addresses", c_void_p), ("down_slots", c_void_p), ("output", c_void_p), ("telemetry", c_void_p),
        ("capacity_rows", c_uint32),
    ]


class WorkReport(ctypes.Structure):
    _fields_ = [
        ("total_ms", c_float), ("stage_ms", c_float * 8), ("gate_up_kernel_ms", c_float),
        ("down_kernel_ms", c_float), ("tensor_path", c_uint32), ("batch_width", c_uint32), ("routes", c_uint32),
        ("distinct_experts", c_uint32), ("kernel_launches", c_uint32), ("weight_bytes_touched", c_uint64),
    ]


class MmaProbe(ctypes.Structure):
    _fields_ = [
        ("n_tile", c_uint32), ("ctas", c_uint32), ("mmas_per_cta", c_uint64), ("elapsed_ms", c_float),
        ("cycles_per_mma", ctypes.c_double), ("tflops", ctypes.c_double), ("sm_clock_mhz_nominal", ctypes.c_double),
    ]


# name -> (restype, argtypes); every symbol the header declares
PROTOTYPES = {
    "nvmoe_geometry_default": (None, [POINTER(Geometry), c_uint32, c_uint32, c_uint32, c_uint32]),
    "nvmoe_device_open": (c_int, [c_int, POINTER(c_void_p)]),
    "nvmoe_device_close": (None, [c_void_p]),
    "nvmoe_last_error": (c_char_p, [c_void_p]),
    "nvmoe_device_stream": (c_void_p, [c_void_p]),
    "nvmoe_buffer_create": (c_int, [c_void_p, c_size_t, POINTER(c_void_p)]),
    "nvmoe_buffer_destroy": (None, [c_void_p]),
    "nvmoe_buffer_write": (c_int, [c_void_p, c_size_t, c_void_p, c_size_t]),
    "nvmoe_buffer_read": (c_int, [c_void_p, c_size_t, c_void_p, c_size_t]),
    "nvmoe_buffer_fill": (c_int, [c_void_p, c_size_t, c_int, c_size_t]),
    "nvmoe_buffer_device_address": (c_uint64, [c_void_p]),
    "nvmoe_buffer_byte_capacity": (c_size_t, [c_void_p]),
    "nvmoe_sync": (c_int, [c_void_p, c_uint64]),
    "nvmoe_plan_create": (c_int, [c_void_p, POINTER(Geometry), POINTER(c_void_p)]),
    "nvmoe_plan_destroy": (None, [c_void_p]),
    "nvmoe_plan_status": (c_int, [c_void_p, POINTER(c_uint32)]),
    "nvmoe_plan_set_expert_path": (c_int, [c_void_p, c_int]),
    "nvmoe_plan_set_profiling": (c_int, [c_void_p, c_int]),
    "nvmoe_buffer_mark_dirty": (c_int, [c_void_p]),
    "nvmoe_plan_set_wait_limit": (c_int, [c_void_p, c_uint64]),
    "nvmoe_plan_debug_withhold_arrival": (c_int, [c_void_p, c_int]),
    "nvmoe_router_linear": (c_int, [c_void_p, c_uint32, c_void_p, c_void_p, c_void_p, c_void_p]),
    "nvmoe_route": (c_int, [c_void_p, c_uint32, c_void_p, c_void_p, c_void_p, c_void_p]),
    "nvmoe_resource_preselect_table": (c_int, [c_void_p, c_uint32, c_void_p, c_void_p, c_void_p, c_uint32, c_uint32, c_void_p]),
    "nvmoe_route_preselected": (c_int, [c_void_p, c_uint32, c_void_p, c_void_p, c_void_p]),
    "nvmoe_rms_norm": (c_int, [c_void_p, c_uint32, c_uint32, c_void_p, c_void_p, c_void_p, c_float, c_float]),
    "nvmoe_silu_multiply": (c_int, [c_void_p, c_uint32, c_uint32, c_void_p, c_void_p, c_void_p, c_float]),
    "nvmoe_residual_add": (c_int, [c_void_p, c_uint32, c_uint32, c_void_p, c_void_p, c_void_p]),
    "nvmoe_dense_linear": (c_int, [c_void_p, c_uint32, c_void_p, c_void_p, c_void_p, c_void_p, c_uint32, c_uint32]),
    "nvmoe_route_compact": (c_int, [c_void_p, c_uint32, c_void_p, c_void_p, c_void_p, c_void_p]),
    "nvmoe_route_compact_static": (c_int, [c_void_p, c_uint32, c_void_p, c_void_p, c_void_p, c_void_p]),
    "nvmoe_route_count": (c_int, [c_void_p, c_uint32, c_void_p, c_void_p, c_void_p]),
    "nvmoe_quantize_fp8": (c_int, [c_void_p, c_uint32, c_uint32, c_void_p, c_void_p, c_void_p]),
    "nvmoe_gate_up": (c_int, [c_void_p, c_uint32, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "nvmoe_gate_up_prequant": (c_int, [c_void_p, c_uint32, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                       c_void_p, c_void_p]),
    "nvmoe_down": (c_int, [c_void_p, c_uint32, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "nvmoe_reduce": (c_int, [c_void_p, c_uint32, c_void_p, c_void_p]),
    "nvmoe_down_partial": (c_int, [c_void_p, c_uint32, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "nvmoe_sum_f32_scale_packed_bf16": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_uint32, c_uint32, c_uint32, c_uint32,
                                                c_uint32]),
    "nvmoe_layer": (c_int, [c_void_p, POINTER(LayerArgs)]),
    "nvmoe_layer_host": (c_int, [c_void_p, POINTER(LayerArgs), c_void_p, c_void_p]),
    "nvmoe_plan_last_report": (c_int, [c_void_p, POINTER(WorkReport)]),
    "nvmoe_plan_launch_count": (c_uint64, [c_void_p]),
    "nvmoe_plan_debug_cta_trace": (c_int, [c_void_p, c_void_p, c_uint32, c_void_p]),
    "nvmoe_plan_debug_counters": (c_int, [c_void_p, POINTER(c_uint64)]),
    "nvmoe_probe_mma_rate": (c_int, [c_void_p, c_uint32, c_uint32, POINTER(MmaProbe)]),
    "nvmoe_buffer_wrap": (c_int, [c_void_p, c_void_p, c_size_t, POINTER(c_void_p)]),
    "nvmoe_device_set_stream": (c_int, [c_void_p, c_void_p]),
    "nvmoe_ep_pack": (c_int, [c_void_p, c_uint32, c_void_p, c_void_p, c_void_p, c_uint32, c_uint32, c_void_p, c_void_p,
                              c_void_p, c_void_p, c_uint32]),
    "nvmoe_ep_unpack": (c_int, [c_void_p, c_uint32, c_void_p, c_void_p, c_void_p]),
    "nvmoe_ep_unique_id": (c_int, [c_void_p]),
    "nvmoe_ep_create": (c_int, [c_void_p, c_void_p, c_uint32, c_uint32, POINTER(c_void_p)]),
    "nvmoe_ep_destroy": (None, [c_void_p]),
    "nvmoe_ep_layer": (c_int, [c_void_p, c_void_p, c_void_p, POINTER(EpLayerArgs)]),
    "nvmoe_ep_sync": (c_int, [c_void_p, c_uint64]),
}

_lib = None


def load() -> ctypes.CDLL:
    """Loads the library and binds every prototype. Raises if it is missing or incomplete."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m nerve_b200.build` (nvcc, sm_100a). "
            "The MoE backend has no CPU fallback."
        )
    lib = ctypes.CDLL(str(LIB_PATH))
    for name, (restype, argtypes) in PROTOTYPES.items():
        fn = getattr(lib, name)  # AttributeError here means the library is stale
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib
