"""Builds libdecide_cuda.so in-tree with nvcc for sm_100a.

`python -m decide_b200.build` compiles every csrc/*.cu to an object file (in parallel, only
when a source or header is newer) and links them into decide_b200/libdecide_cuda.so. nvcc
cross-compiles without a GPU, so this also runs on a CPU-only machine.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OBJ = PKG / "build"
LIB = PKG / "libdecide_cuda.so"
INCLUDE = PKG.parent / "include"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
    "-Xptxas", "-v",
]


def source_files() -> list[tuple[str, Path]]:
    """The files the library is built from, as sorted (relative name, path): every csrc/*.cu and *.cuh and the public header."""
    files = [(f"csrc/{p.name}", p) for p in list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh"))] + [(f"include/{p.name}", p) for p in INCLUDE.glob("*.h")]
    return sorted(files)


def source_hash() -> str:
    """Content hash of the kernel sources, the reference's stale-binary guard (crates/decide-metal/src/source_hash.rs:47-62):
    FNV-1a 64 over `relative path NUL contents NUL` in sorted path order, as 16 hex digits. The library carries the hash of
    the sources it was built from (dc_source_hash); decide_b200._lib refuses a library whose hash is not the sources'."""
    h = 0xCBF29CE484222325
    for rel, path in source_files():
        for chunk in (rel.encode(), b"\0", path.read_bytes(), b"\0"):
            for b in chunk:
                h = ((h ^ b) * 0x100000001B3) & 0xFFFFFFFFFFFFFFFF
    return f"{h:016x}"


def nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: the CUDA kernels cannot be built")
    return exe


def _newest_header() -> float:
    headers = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + list(INCLUDE.glob("*.h"))
    return max(p.stat().st_mtime for p in headers)


def _compile(src: Path, force: bool, header_time: float) -> tuple[Path, str]:
    obj = OBJ / (src.stem + ".o")
    if not force and obj.exists() and obj.stat().st_mtime >= max(src.stat().st_mtime, header_time):
        return obj, ""
    cmd = [nvcc(), *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stdout}\n{r.stderr}")
    return obj, r.stderr


def build(force: bool = False, verbose: bool = False) -> Path:
    OBJ.mkdir(exist_ok=True)
    sources = sorted(CSRC.glob("*.cu"))
    header_time = _newest_header()
    with ThreadPoolExecutor(max_workers=min(8, len(sources))) as pool:
        results = list(pool.map(lambda s: _compile(s, force, header_time), sources))
    objs = [o for o, _ in results]
    # the stamp: a generated translation unit holding the hash of the sources above
    digest = source_hash()
    stamp_src, stamp_obj = OBJ / "source_hash_stamp.cu", OBJ / "source_hash_stamp.o"
    text = f'extern "C" const char* dc_source_hash() {{ return "{digest}"; }}\n'
    if not stamp_src.exists() or stamp_src.read_text() != text or not stamp_obj.exists():
        stamp_src.write_text(text)
        r = subprocess.run([nvcc(), "-O1", "-Xcompiler", "-fPIC", "-c", str(stamp_src), "-o", str(stamp_obj)], capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for the source-hash stamp:\n{r.stdout}\n{r.stderr}")
    objs.append(stamp_obj)
    if verbose:
        for _, log in results:
            if log:
                sys.stderr.write(log)
    if force or not LIB.exists() or any(o.stat().st_mtime > LIB.stat().st_mtime for o in objs):
        cmd = [nvcc(), "-shared", "-o", str(LIB), *map(str, objs), "-gencode", "arch=compute_100a,code=sm_100a", "-ldl"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose=True)
    print(path)
