#!/usr/bin/env python
"""Prints the Rust ``extern "C"`` block for ``singe-kernel-sys/src/lib.rs`` from ``singe_kernel_sys.h``.

``python include/rust_bindings.py`` writes one declaration per function the header declares, with the C types mapped
one to one (pointers stay raw: the safe wrappers live in ``singe-kernel``, which already owns the typed device
buffers).  No Rust toolchain is needed to run it.
"""
from __future__ import annotations

import os
import re

HERE = os.path.dirname(os.path.abspath(__file__))

TYPES = {
    "singe_stream_t": "SingeStream",
    "size_t": "usize",
    "int": "c_int",
    "unsigned": "c_uint",
    "float": "f32",
    "int64_t": "i64",
    "void *": "*mut c_void",
    "const void *": "*const c_void",
    "void **": "*mut *mut c_void",
    "void *const *": "*const *mut c_void",
    "const void *const *": "*const *const c_void",
    "float *": "*mut f32",
    "const float *": "*const f32",
    "int64_t *": "*mut i64",
    "const int32_t *": "*const i32",
    "uint32_t *": "*mut u32",
    "const uint32_t *": "*const u32",
    "uint32_t *const *": "*const *mut u32",
}
RETURNS = {"int": " -> c_int", "size_t": " -> usize", "const char *": " -> *const c_char", "void": ""}
KEYWORDS = {"where": "at", "type": "kind", "in": "input", "ref": "reference", "match": "matched", "loop": "looped"}


def declarations(header: str):
    text = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    pattern = r"\n((?:int|size_t|const char \*|void)\s*)(singe_[a-z0-9_]+)\s*\(([^;]*)\);"
    for returned, name, arguments in re.findall(pattern, text):
        fields = []
        for argument in arguments.split(","):
            argument = " ".join(argument.split())
            if argument in ("", "void"):
                continue
            kind, identifier = re.match(r"(.*?)(\w+)$", argument).groups()
            fields.append((KEYWORDS.get(identifier, identifier), TYPES[kind.strip()]))
        yield name, fields, RETURNS[returned.strip()]


def render() -> str:
    with open(os.path.join(HERE, "singe_kernel_sys.h")) as handle:
        header = handle.read()
    lines = ["use core::ffi::{c_char, c_int, c_uint, c_void};", "",
             "/// A `CUstream` / `cudaStream_t`.", "pub type SingeStream = *mut c_void;", "",
             '#[link(name = "singe_kernel_sys")]', 'unsafe extern "C" {']
    for name, fields, returned in declarations(header):
        arguments = ", ".join(f"{identifier}: {kind}" for identifier, kind in fields)
        lines.append(f"    pub fn {name}({arguments}){returned};")
    lines.append("}")
    return "\n".join(lines) + "\n"


if __name__ == "__main__":
    print(render(), end="")
