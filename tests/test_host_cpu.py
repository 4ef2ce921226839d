"""CPU-side checks of the product: the library loads, exports every declared symbol, and the
host logic that needs no GPU behaves (no compute calls are made here)."""
import ctypes
import re
from pathlib import Path

import numpy as np
import pytest

from nerve_b200 import capi, synthetic

ROOT = Path(__file__).resolve().parent.parent


def test_library_exports_every_symbol_the_header_declares():
    lib = capi.load()
    header = (ROOT / "include" / "nerve_cuda_moe.h").read_text()
    declared = set(re.findall(r"^(?:int|void|const char\*|void\*|uint64_t|size_t)\s+(nvmoe_[a-z0-9_]+)\(", header, re.M))
    assert declared, "no declarations found"
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
        assert name in capi.PROTOTYPES, f"{name} has no ctypes prototype"


def test_struct_layouts_match_the_header():
    # sizes follow from the field lists in include/nerve_cuda_moe.h
    assert ctypes.sizeof(capi.Geometry) == 23 * 4
    assert ctypes.sizeof(capi.LayerArgs) == 3 * 4 + 4 + 14 * 8
    assert ctypes.sizeof(capi.WorkReport) == 4 + 8 * 4 + 3 * 4 + 4 * 4 + 8
    assert ctypes.sizeof(capi.EpLayerArgs) == 4 + 4 + 11 * 8 + 8


def test_expert_parallel_entry_points_reject_bad_arguments_without_a_gpu():
    lib = capi.load()
    assert lib.nvmoe_ep_unique_id(None) != 0
    handle = ctypes.c_void_p()
    assert lib.nvmoe_ep_create(None, b"\0" * 128, 0, 1, ctypes.byref(handle)) != 0
    assert lib.nvmoe_ep_layer(None, None, None, None) != 0
    lib.nvmoe_ep_destroy(None)  # a null handle is ignored


def test_geometry_default_matches_reference_constants():
    g = capi.Geometry()
    capi.load().nvmoe_geometry_default(ctypes.byref(g), 4096, 2048, 256, 6)
    # nerve/model_package_independent_experts.py:17-18 and the 128-column activation block
    assert (g.gate_tile_rows, g.down_tile_rows, g.act_block) == (32, 64, 128)
    assert g.swiglu_alpha == 1.0 and g.swiglu_up_offset == 0.0 and g.n_group == 0
    assert g.reduce_scale == 1.0 and g.routed_scale == 1.0


def test_device_open_without_a_gpu_reports_an_error():
    torch = pytest.importorskip("torch")
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    lib = capi.load()
    handle = ctypes.c_void_p()
    rc = lib.nvmoe_device_open(0, ctypes.byref(handle))
    assert rc != 0 and not handle.value
    assert lib.nvmoe_last_error(None)


def test_synthetic_cases_are_seeded_and_shaped():
    cfg = synthetic.small_variant(synthetic.CONFIGS["gpt-oss-20b"], 64, 96, 8)
    a = synthetic.make_case(cfg, 5, seed=3)
    b = synthetic.make_case(cfg, 5, seed=3)
    c = synthetic.make_case(cfg, 5, seed=4)
    assert np.array_equal(a.hidden, b.hidden) and not np.array_equal(a.hidden, c.hidden)
    assert a.w1[0].shape == (96, 32) and a.s1[0].shape == (96, 2) and a.w2[0].shape == (64, 48)
    assert a.s1[0].min() >= 121 and a.s1[0].max() <= 127
    assert synthetic.CONFIGS["gpt-oss-20b"].expert_weight_bytes == 13_219_200
    assert synthetic.CONFIGS["deepseek-v3"].expert_weight_bytes == 23_396_352
    assert synthetic.CONFIGS["tiny"].expert_weight_bytes == 208_896


def test_public_headers_compile_as_plain_c(tmp_path):
    """The boundary is a C ABI: both headers must be valid C99 on their own."""
    import shutil
    import subprocess

    gcc = shutil.which("gcc") or "/usr/bin/gcc"
    source = tmp_path / "abi.c"
    source.write_text(
        '#include "nerve_cuda_moe.h"\n#include "nvmoe_math.h"\n'
        "int main(void) { nvmoe_geometry g; nvmoe_layer_args a; nvmoe_ep_layer_args e; nvmoe_work_report r;\n"
        "  (void)g; (void)a; (void)e; (void)r; return nvmoe_expf(0.0f) == 1.0f ? 0 : 1; }\n")
    include = Path(__file__).resolve().parent.parent / "include"
    binary = tmp_path / "abi"
    subprocess.run([gcc, "-std=c99", "-Wall", "-Wextra", "-Werror", "-pedantic", "-ffp-contract=off", f"-I{include}",
                    str(source), "-o", str(binary), "-lm"], check=True)
    subprocess.run([str(binary)], check=True)

