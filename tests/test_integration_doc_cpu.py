"""The binding a maintainer would paste from INTEGRATION.md must be the one the header implies:
the Rust `extern "C"` block there is compared with what nerve_b200.rust_binding writes from
include/nerve_cuda_moe.h, and the parsed prototypes with the ctypes prototypes the tests call through."""
import re
from pathlib import Path

from nerve_b200 import capi, rust_binding

ROOT = Path(__file__).resolve().parent.parent


def test_parsed_prototypes_cover_the_header_and_agree_with_ctypes():
    header = (ROOT / "include" / "nerve_cuda_moe.h").read_text()
    declared = set(re.findall(r"^(?:int|void|const char\*|void\*|uint64_t|size_t)\s+(nvmoe_[a-z0-9_]+)\(", header, re.M))
    _, structs, functions = rust_binding.parse()
    names = {name for name, _, _ in functions}
    assert names == declared
    for name, _, params in functions:
        _, argtypes = capi.PROTOTYPES[name]
        assert len(argtypes) == len(params), f"{name}: header has {len(params)} parameters, ctypes {len(argtypes)}"
    sizes = {name: len(fields) for name, fields in structs}
    assert sizes["nvmoe_geometry"] == 23 and "nvmoe_layer_args" in sizes and "nvmoe_ep_layer_args" in sizes


def test_rust_types():
    assert rust_binding.rust_type("const nvmoe_buffer*") == "*const nvmoe_buffer"
    assert rust_binding.rust_type("nvmoe_plan**") == "*mut *mut nvmoe_plan"
    assert rust_binding.rust_type("const void*") == "*const c_void"
    assert rust_binding.rust_type("uint64_t") == "u64"


def test_integration_guide_carries_the_generated_binding():
    text = (ROOT / "INTEGRATION.md").read_text()
    blocks = [b for b in re.findall(r"```rust\n(.*?)```", text, re.S) if 'extern "C" {' in b]
    assert len(blocks) == 1, "INTEGRATION.md must hold exactly one extern block"
    assert blocks[0] == rust_binding.render(), "regenerate the block: python -m nerve_b200.rust_binding"
    # the one prototype an earlier version of the guide had wrong
    assert "pub fn nvmoe_geometry_default(g: *mut nvmoe_geometry, hidden: u32, intermediate: u32, experts: u32, k: u32);" in blocks[0]
