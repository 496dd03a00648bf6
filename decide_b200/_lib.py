"""ctypes binding of libdecide_cuda.so.

Prototypes are read out of include/decide_cuda.h, so the header stays the single definition of
the ABI: every `int|uint32_t|... dc_xxx(...)` declaration becomes a typed ctypes function. There
is no fallback: if the shared library is missing, `load()` raises.
"""
from __future__ import annotations

import ctypes
import os
import re
from pathlib import Path

PKG = Path(__file__).resolve().parent
HEADER = PKG.parent / "include" / "decide_cuda.h"
LIB_PATH = PKG / "libdecide_cuda.so"

_CTYPES = {
    "int": ctypes.c_int,
    "uint32_t": ctypes.c_uint32,
    "uint64_t": ctypes.c_uint64,
    "size_t": ctypes.c_size_t,
    "float": ctypes.c_float,
    "void": None,
}


def _ctype(decl: str):
    """C parameter/return type text -> ctypes type. Every pointer is passed as void*."""
    decl = decl.replace("const", " ").strip()
    if "*" in decl:
        return ctypes.c_void_p
    base = decl.split()[0]
    return _CTYPES[base]


def header_prototypes(text: str | None = None) -> dict[str, tuple]:
    """{name: (restype, [argtypes], [argnames])} for every function the header declares."""
    text = HEADER.read_text() if text is None else text
    text = re.sub(r"/\*.*?\*/", " ", text, flags=re.S)
    text = re.sub(r"^[ \t]*#.*$", " ", text, flags=re.M)   # preprocessor lines are not declarations
    protos = {}
    for m in re.finditer(r"([A-Za-z_][\w\s\*]*?)\b(dc_\w+)\s*\(([^;{}]*?)\)\s*;", text):
        ret, name, params = m.group(1).strip(), m.group(2), m.group(3).strip()
        argtypes, argnames = [], []
        if params and params != "void":
            for p in params.split(","):
                p = " ".join(p.split())
                argnames.append(re.split(r"[\s\*]+", p)[-1])
                argtypes.append(_ctype(p.rsplit(argnames[-1], 1)[0] + ("*" if "*" in p else "")))
        protos[name] = (_ctype(ret + " "), argtypes, argnames)
    return protos


_lib = None


def load() -> ctypes.CDLL:
    """Loads the library once and types every exported function. Raises if it is not built."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is not built (run `python -m decide_b200.build`); decide_b200 has no CPU fallback")
    lib = ctypes.CDLL(str(LIB_PATH))
    for name, (restype, argtypes, _) in header_prototypes().items():
        fn = getattr(lib, name)  # AttributeError here = the header declares a symbol the library lacks
        fn.restype = restype
        fn.argtypes = argtypes
    # The stale-binary guard of the reference (crates/decide-metal/src/source_hash.rs, lib.rs:18-21): the library carries the
    # hash of the sources it was built from and is refused when the sources beside it have changed since.
    lib.dc_source_hash.restype = ctypes.c_char_p
    built_from = lib.dc_source_hash().decode()
    from . import build

    if (PKG / "csrc").is_dir() and not os.environ.get("DECIDE_ALLOW_STALE_LIBRARY"):
        now = build.source_hash()
        if now != built_from:
            raise RuntimeError(f"{LIB_PATH} was built from other sources (hash {built_from}, the sources hash to {now}): "
                               "run `python -m decide_b200.build` (DECIDE_ALLOW_STALE_LIBRARY=1 overrides)")
    _lib = lib
    return lib
