"""Generates src/ffi.rs from include/decide_cuda.h, one `pub fn` per declared `dc_*` function.

    python crates/decide-cuda/gen_ffi.py            # rewrites crates/decide-cuda/src/ffi.rs

The header is the single definition of the ABI; the Python binding types its prototypes from it at
import time (decide_b200/_lib.py) and this script does the same for Rust. tests/test_abi.py checks
that the committed ffi.rs is what this script produces from the committed header.
"""
import re
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[2]
HEADER = ROOT / "include" / "decide_cuda.h"
OUT = Path(__file__).resolve().parent / "src" / "ffi.rs"

SCALARS = {"int": "i32", "uint32_t": "u32", "uint64_t": "u64", "size_t": "usize", "float": "f32", "char": "c_char", "void": "c_void",
           "dc_ctx": "DcCtx", "dc_model": "DcModel", "dc_dims": "DcDims", "dc_layer_weights": "DcLayerWeights", "dc_convert_report": "DcConvertReport"}
KEYWORDS = {"type", "ref", "in", "impl", "mod", "move", "fn", "match", "loop", "where"}


def rust_type(c: str) -> str:
    c = " ".join(c.split())
    const = "const" in c.split()
    base = c.replace("const", " ").replace("*", " ").split()[0]
    stars = c.count("*")
    t = SCALARS[base]
    for _ in range(stars):
        t = ("*const " if const else "*mut ") + t
    return t


def prototypes(text: str):
    text = re.sub(r"/\*.*?\*/", " ", text, flags=re.S)
    text = re.sub(r"^[ \t]*#.*$", " ", text, flags=re.M)
    for m in re.finditer(r"([A-Za-z_][\w\s\*]*?)\b(dc_\w+)\s*\(([^;{}]*?)\)\s*;", text):
        ret, name, params = m.group(1).strip(), m.group(2), m.group(3).strip()
        args = []
        if params and params != "void":
            for p in params.split(","):
                p = " ".join(p.split())
                arg = re.split(r"[\s\*]+", p)[-1]
                ctype = p[: p.rfind(arg)]
                args.append((arg + "_" if arg in KEYWORDS else arg, rust_type(ctype)))
        yield name, args, (None if ret == "void" else rust_type(ret))


def render() -> str:
    lines = ["//! Raw bindings of libdecide_cuda.so: GENERATED from include/decide_cuda.h by gen_ffi.py; do not edit.",
             "//! Not compiled in the image this crate was written in (no Rust toolchain there): unverified.",
             "#![allow(clippy::too_many_arguments)]", "use std::os::raw::{c_char, c_void};", "",
             "#[repr(C)] pub struct DcCtx { _private: [u8; 0] }", "#[repr(C)] pub struct DcModel { _private: [u8; 0] }", "",
             "/// dc_convert_report: the converter's fp16 precision-loss counters.",
             "#[repr(C)] #[derive(Clone, Copy, Debug, Default, PartialEq, Eq)]",
             "pub struct DcConvertReport { pub values: u64, pub f16_subnormal: u64, pub f16_flushed_to_zero: u64, pub f16_overflow: u64 }", "",
             "/// dc_dims: the model's dims, compile-time constants in the reference (config.rs:4-37).",
             "#[repr(C)] #[derive(Clone, Copy, Debug, PartialEq)]",
             "pub struct DcDims {", "    pub hidden: u32, pub n_layers: u32, pub nq: u32, pub nkv: u32, pub head_dim: u32, pub rot_dim: u32,",
             "    pub gdn_nk: u32, pub gdn_nv: u32, pub gdn_dk: u32, pub gdn_dv: u32, pub inter: u32, pub vocab: u32,",
             "    pub full_attn_interval: u32, pub attn_gate: u32, pub swiglu_block: u32, pub eps: f32, pub rope_theta: f32,", "}", "",
             "/// dc_layer_weights: one layer's device pointers in the fused layouts (convert.rs:204-245); unused members null.",
             "#[repr(C)] #[derive(Clone, Copy, Debug)]",
             "pub struct DcLayerWeights {", "    pub in_norm: *const f32, pub w_in: *const c_void, pub w_out: *const c_void, pub post_norm: *const f32,",
             "    pub w_gu: *const c_void, pub w_down: *const c_void, pub conv_w: *const f32, pub a_log: *const f32, pub dt_bias: *const f32,",
             "    pub gnorm: *const f32, pub q_norm: *const f32, pub k_norm: *const f32,", "}", "",
             "pub const DC_OK: i32 = 0;", "pub const DC_INVALID_ARG: i32 = 1;", "pub const DC_CUDA_ERROR: i32 = 2;", "pub const DC_UNSUPPORTED: i32 = 3;",
             "pub const DC_TIMEOUT: i32 = 4;", "pub const DC_NOALLOC_MAX_VALUES: u64 = 1 << 32;", "pub const DC_GEMM_SMALL_MAX_M: u32 = 16;", "",
             '#[link(name = "decide_cuda")]', 'extern "C" {']
    for name, args, ret in prototypes(HEADER.read_text()):
        sig = ", ".join(f"{a}: {t}" for a, t in args)
        lines.append(f"    pub fn {name}({sig}){' -> ' + ret if ret else ''};")
    lines += ["}", ""]
    return "\n".join(lines)


if __name__ == "__main__":
    if "--check" in sys.argv:
        sys.exit(0 if OUT.read_text() == render() else 1)
    OUT.write_text(render())
    print(OUT)
