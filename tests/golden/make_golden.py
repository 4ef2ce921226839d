"""Regenerates the golden fixtures in this folder from the importable Python half of the reference.

Run once, in a container that has the reference checkout (it cannot travel to a GPU box):

    PYTHONPATH=<reference checkout> python tests/golden/make_golden.py

What is taken from the reference itself (imported and executed, nothing copied):
  * nerve.quantized_transforms — the E2M1 -> SINT8 and E2M1 -> E4M3 tables, the exact rational
    value of every (nibble, E8M0 byte) pair, and every finite E4M3 byte
    (tests/test_quantized_transforms.py:22-50 are the reference's own checks of these);
  * the numpy MXFP4 decoder PackageTensorRepository._decode_mxfp4 / _e8m0_to_f32
    (nerve/representation_optimizer/analysis/tensor_repository.py:472-547,769-773) run on a seeded
    random packed tensor through the same package scaffold its own test uses
    (tests/test_analysis_tensor_repository.py:21-63,264-338);
  * independent_sparse_moe_body (nerve/circuit_lowering_sparse_experts.py:7-212): the node chain,
    binding-relevant attributes and signal names the C ABI mirrors.

What is transcribed as data from the reference's GPU-only Rust tests (they need a Vulkan device
and cannot run here): the constant-fill known answers and control words of
runtime-rs/src/vulkan_compute/mxfp4_tests.rs:89-215,279-313 and
runtime-rs/src/vulkan_compute/mxfp4_route_native_tests.rs:57-65,237-249,297-303.
"""
from __future__ import annotations

import json
import struct
import sys
import tempfile
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent


def tables() -> dict:
    from nerve import quantized_transforms as qt

    values = {}
    for scale in range(0xFF):
        for nibble in range(16):
            v = qt.mxfp4_value(nibble, scale)
            values[f"{nibble}:{scale}"] = [v.numerator, v.denominator]
    e4m3 = {}
    for bits in range(256):
        v = qt.fp8_e4m3_value(bits)
        e4m3[str(bits)] = [v.numerator, v.denominator]
    return {
        "sint8_codes": list(qt.MXFP4_E2M1_SINT8_CODES),
        "e4m3_bits": list(qt.MXFP4_E2M1_FP8_E4M3_BITS),
        "expand_sint8": {"input": [0x10, 0x87, 0xFE],
                         "output": list(qt.expand_mxfp4_e2m1_to_sint8(bytes((0x10, 0x87, 0xFE))))},
        "expand_e4m3": {"input": [0x10, 0xF8],
                        "output": list(qt.expand_mxfp4_e2m1_to_fp8_e4m3(bytes((0x10, 0xF8))))},
        "mxfp4_value": values,
        "e4m3_value": e4m3,
        "e8m0": {str(b): [qt.e8m0_scale(b).numerator, qt.e8m0_scale(b).denominator] for b in range(0xFF)},
    }


def numpy_decoder() -> dict:
    from nerve.representation_optimizer.analysis.tensor_repository import PackageTensorRepository

    rng = np.random.Generator(np.random.PCG64(20240611))
    rows, cols = 6, 96
    packed = rng.integers(0, 256, (rows, cols // 2), dtype=np.uint8)
    scales = rng.integers(110, 135, (rows, cols // 32), dtype=np.uint8)
    scales[0, 0] = 0  # the 2^-127 special case
    records = [
        ("w", "I8", [rows, cols // 2], packed.tobytes(), {
            "logical_shape": [rows, cols],
            "quantization": {
                "format": "mxfp4_e2m1", "bits": 4, "element_type": "float", "values_per_byte": 2,
                "packing_axis": 1, "packing_order": "low_nibble_then_high_nibble_along_k",
                "group_size": 32, "scales": "w_scale", "scale_dtype": "F8_E8M0",
                "scale_mode": "power_of_two_per_output_row_k_group",
            },
        }),
        ("w_scale", "F8_E8M0", [rows, cols // 32], scales.tobytes(), {}),
    ]
    with tempfile.TemporaryDirectory() as tmp:
        root = Path(tmp)
        header, payload, tensors = {}, bytearray(), {}
        for name, dtype, shape, data, ext in records:
            start = len(payload)
            payload.extend(data)
            stop = len(payload)
            header[name] = {"dtype": dtype, "shape": shape, "data_offsets": [start, stop]}
            ext = dict(ext)
            tensors[name] = {"dtype": dtype, "shape": shape,
                             "logical_shape": ext.pop("logical_shape", shape),
                             "source_file": "weights/test.safetensors",
                             "data_offsets": [start, stop], **ext}
        header_bytes = json.dumps(header, separators=(",", ":")).encode()
        source = root / "weights" / "test.safetensors"
        source.parent.mkdir(parents=True)
        source.write_bytes(struct.pack("<Q", len(header_bytes)) + header_bytes + payload)
        index = {"tensors": tensors, "source": {"weights_files": [
            {"path": "weights/test.safetensors", "safetensors_header_bytes": len(header_bytes)}]}}
        repo = PackageTensorRepository(root, index)
        observed = repo.observe("w", exhaustive_element_limit=None, sampled_element_limit=64)
        decoded = np.asarray(observed.values, dtype=np.float32)
    return {
        "rows": rows, "cols": cols,
        "packed": packed.reshape(-1).tolist(),
        "scales": scales.reshape(-1).tolist(),
        "decoded_f32_bits": decoded.view(np.uint32).reshape(-1).tolist(),
    }


def node_chain() -> dict:
    """The node lists the compiler emits for the route-native MoE body (score-selected routing, and the
    token-id-table form with its preselection node), with the packaged weight + scale parameter pairs."""
    from nerve.circuit_lowering_sparse_experts import independent_sparse_moe_body

    experts = list(range(4))
    parameters = {"moe_router": {}, "moe_router_selection_bias": {}, "moe_route_table": {}}
    for e in experts:
        for proj in ("w1", "w2", "w3"):
            parameters[f"routed_expert_{e:03d}_{proj}"] = {}
            parameters[f"routed_expert_{e:03d}_{proj}_scale"] = {}
    for proj in ("w1", "w2", "w3"):
        parameters[f"shared_expert_{proj}"] = {}
        parameters[f"shared_expert_{proj}_scale"] = {}

    def chain(selection: str) -> list:
        feed_forward = {
            "routing": {"selection": selection, "activation": "sigmoid", "normalize_selected": True,
                        "routed_scaling_factor": 2.5},
            "expert_ids": experts, "intermediate_size": 128, "hidden_size": 128,
            "experts_per_token": 2, "swiglu_limit": 10.0,
        }
        body = independent_sparse_moe_body(feed_forward=feed_forward, parameters=parameters)
        return [{"id": n["id"], "op": n["op"], "inputs": n["inputs"], "outputs": n["outputs"],
                 "params": n.get("params", []), "attrs": n.get("attrs", {})} for n in body]

    return {"nodes": chain("score_topk"), "token_id_table_nodes": chain("token_id_table")}


def rust_known_answers() -> dict:
    """Data of the reference's Vulkan-only conformance tests, transcribed by reading them."""
    return {
        "constant_fill": {  # mxfp4_tests.rs:5-8,89-132,164-215
            "width": 128, "weight_fill": 0x22, "scale_fill": 120, "route_weight": 1.0,
            "swiglu_limit": 10.0, "gate_tile_rows": 32, "down_tile_rows": 64,
            "gate_up_expected": "bf16(1/(1+exp(-1)))", "down_expected": 1.0,
            "e2m1_values": [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0,
                            0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0],
            "prequant_hidden_byte": 0x38, "prequant_scale": 1.0,
        },
        "fail_closed": {  # mxfp4_tests.rs:279-313
            "invalid_compact_route": 0xFFFFFFFF, "zeroed_address_table_leaves_zeros": True,
        },
        "route_native": {  # mxfp4_route_native_tests.rs:11-14,57-65,69-101,237-249
            "hidden": 128, "intermediate": 128, "experts": 4, "k": 2,
            "routes": [[3, 0.75], [1, 0.25]], "bound_experts": [1, 3],
            "fills": {"1": 0x22, "3": 0x44}, "scale_fill": 120,
            "control_in": [1, 0, 4, 0, 0, 0, 0],
            "gate_control_out": [1, 0, 4, 2, 8, 1, 1],
            "down_control_out": [1, 0, 4, 2, 4, 1, 1],
            "canonical_control": {"gate": [1, 0, 0, 0, 8, 1, 1], "down": [1, 0, 0, 0, 4, 1, 1]},
        },
        "tp_reduction": {  # mxfp4_route_native_tests.rs:297-303,410-433
            "intermediate_word_base": 0x3C384030, "reduction_push": [256, 1, 1, 128, 16],
        },
        "port_shapes": {  # stream_plan/shape_inference/node_shapes.rs:345-373
            "moe_route": "[K,2]", "gate_up": "[K*I + 2K]", "down": "[K,H]", "reduce": "[H]",
        },
    }


def main() -> None:
    out = {
        "tables": tables(),
        "numpy_decoder": numpy_decoder(),
        "node_chain": node_chain(),
        "rust_known_answers": rust_known_answers(),
    }
    (HERE / "reference_vectors.json").write_text(json.dumps(out, separators=(",", ":")))
    print("wrote", HERE / "reference_vectors.json", (HERE / "reference_vectors.json").stat().st_size, "bytes")


if __name__ == "__main__":
    sys.exit(main())
