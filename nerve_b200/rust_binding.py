"""Writes the Rust `extern "C"` block for include/nerve_cuda_moe.h.

The reference's runtime is Rust (runtime-rs/src/vulkan_compute/compute_device_dispatch.rs:2-273 is the
device object this library stands in for); a maintainer adds one `ffi.rs` with the declarations below and
keeps it in step with the header by re-running this module:

    python -m nerve_b200.rust_binding > runtime-rs/src/cuda_moe/ffi.rs

Only the header's own text is read: opaque handle types, `typedef struct` bodies of plain scalar and
pointer fields, and the function prototypes.  Enumerations are plain `u32`/`c_int` values on the Rust side.
"""
from __future__ import annotations

import re
from pathlib import Path

HEADER = Path(__file__).resolve().parent.parent / "include" / "nerve_cuda_moe.h"

SCALARS = {
    "void": "c_void", "char": "c_char", "int": "c_int", "float": "f32", "double": "f64", "size_t": "usize",
    "uint8_t": "u8", "uint16_t": "u16", "uint32_t": "u32", "uint64_t": "u64", "int32_t": "i32", "int64_t": "i64",
}


def strip_comments(text: str) -> str:
    text = re.sub(r"/\*.*?\*/", " ", text, flags=re.S)
    return re.sub(r"//[^\n]*", " ", text)


def rust_type(c_type: str) -> str:
    """`const nvmoe_buffer*` -> `*const nvmoe_buffer`, `uint32_t` -> `u32`, `void**` -> `*mut *mut c_void`."""
    tokens = c_type.replace("*", " * ").split()
    out, const_pending, base = "", False, None
    for tok in tokens:
        if tok == "const":
            const_pending = True
        elif tok == "struct":
            continue
        elif tok == "*":
            out = ("*const " if const_pending else "*mut ") + out
            const_pending = False
        else:
            base = SCALARS.get(tok, tok)
    assert base is not None, c_type
    return out + base


def split_declarator(decl: str) -> tuple[str, str, int]:
    """`const uint32_t* name[4]` -> (type, name, array length or 0)."""
    decl = decl.strip()
    m = re.match(r"^(.*?)([A-Za-z_][A-Za-z0-9_]*)\s*(?:\[\s*([A-Za-z0-9_]+)\s*\])?$", decl, re.S)
    assert m, decl
    return m.group(1).strip(), m.group(2), m.group(3) or ""


def constants(text: str) -> dict[str, int]:
    """Enumerators with literal values and #define'd integers (array lengths refer to them)."""
    out = {}
    for name, value in re.findall(r"#define\s+([A-Z][A-Z0-9_]*)\s+(\d+)u?\b", text):
        out[name] = int(value)
    for body in re.findall(r"enum\s*(?:[a-z_0-9]+\s*)?\{(.*?)\}", text, re.S):
        nxt = 0
        for item in body.split(","):
            item = item.strip()
            if not item:
                continue
            if "=" in item:
                name, value = [s.strip() for s in item.split("=", 1)]
                m = re.match(r"^(\d+)u?(?:\s*<<\s*(\d+))?$", value)
                if not m:
                    continue
                nxt = int(m.group(1)) << int(m.group(2) or 0)
            else:
                name = item
            out[name] = nxt
            nxt += 1
    return out


def parse(text: str | None = None):
    text = strip_comments(HEADER.read_text() if text is None else text)
    consts = constants(text)
    opaque = re.findall(r"typedef\s+struct\s+([a-z_0-9]+)\s+\1\s*;", text)
    structs = []
    for name, body in re.findall(r"typedef\s+struct\s+([a-z_0-9]+)\s*\{(.*?)\}\s*\1\s*;", text, re.S):
        fields = []
        for decl in body.split(";"):
            if not decl.strip():
                continue
            c_type, first, length = split_declarator(decl.split(",")[0])
            names = [(first, length)] + [split_declarator(c_type + " " + d)[1:] for d in decl.split(",")[1:]]
            for field, n in names:
                fields.append((field, c_type, int(consts.get(n, n)) if n else 0))
        structs.append((name, fields))
    functions = []
    for ret, name, args in re.findall(r"^([A-Za-z_][A-Za-z0-9_ ]*?[\s\*]+)(nvmoe_[a-z0-9_]+)\s*\(([^;{]*?)\)\s*;", text, re.M | re.S):
        params = []
        if args.strip() and args.strip() != "void":
            for arg in args.split(","):
                c_type, pname, _ = split_declarator(arg)
                params.append((pname, c_type))
        functions.append((name, ret.strip(), params))
    return opaque, structs, functions


def render(text: str | None = None) -> str:
    opaque, structs, functions = parse(text)
    lines = ["#![allow(non_camel_case_types)]", "use std::os::raw::{c_char, c_int, c_void};", ""]
    for name in opaque:
        lines.append(f"#[repr(C)] pub struct {name} {{ _p: [u8; 0] }}")
    for name, fields in structs:
        lines += ["", "#[repr(C)] #[derive(Clone, Copy)]", f"pub struct {name} {{"]
        for field, c_type, length in fields:
            t = rust_type(c_type)
            lines.append(f"    pub {field}: {f'[{t}; {length}]' if length else t},")
        lines.append("}")
    lines += ["", 'extern "C" {']
    for name, ret, params in functions:
        args = ", ".join(f"{'r#type' if p == 'type' else p}: {rust_type(t)}" for p, t in params)
        tail = "" if ret == "void" else f" -> {rust_type(ret)}"
        lines.append(f"    pub fn {name}({args}){tail};")
    lines.append("}")
    return "\n".join(lines) + "\n"


if __name__ == "__main__":
    print(render(), end="")
