"""The C ABI surface without a GPU: the library loads, exports every symbol the header declares,
and the host-only entry points behave (no compute calls here)."""
import ctypes

import pytest

from decide_b200 import _lib


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    protos = _lib.header_prototypes()
    assert len(protos) >= 20
    for name in protos:
        assert hasattr(lib, name), f"{name} is declared in include/decide_cuda.h but not exported"


def test_header_parser_types():
    protos = _lib.header_prototypes("int dc_x(dc_ctx* ctx, const float* a, uint32_t n, float eps);\nuint64_t dc_y(void);")
    assert protos["dc_x"][1] == [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint32, ctypes.c_float]
    assert protos["dc_x"][0] is ctypes.c_int
    assert protos["dc_y"] == (ctypes.c_uint64, [], [])


def test_null_context_is_refused_not_dereferenced():
    lib = _lib.load()
    assert lib.dc_gemm(None, None, None, None, None, 1, 32, 32, 32, 32, 32, 0, 16) == 1
    assert lib.dc_launch_count(None) == 0
    lib.dc_close(None)


def test_open_without_a_gpu_fails_loudly():
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    lib = _lib.load()
    err = ctypes.create_string_buffer(256)
    assert not lib.dc_open(0, err, len(err))
    assert b"no CUDA device" in err.value
    from decide_b200.kernels import Device

    with pytest.raises(RuntimeError):
        Device(0)


def test_gemm_plan_covers_engine_shapes():
    """The tile plan answers for every engine shape x row count (the reference checks the same of
    gemm_configs::plan, crates/decide-metal/src/gemm_configs.rs:386-401)."""
    lib = _lib.load()
    for n in (19456, 2560, 8224, 6144, 10240):
        for m in (1, 8, 16, 163, 276, 603, 2307, 38592):
            assert lib.dc_gemm_plan(None, m, n) in (128, 192, 224, 256)


def test_rust_ffi_is_generated_from_the_header():
    """crates/decide-cuda/src/ffi.rs is what crates/decide-cuda/gen_ffi.py makes of include/decide_cuda.h: one `pub fn` per
    declared dc_* function, so the (uncompiled) Rust binding cannot drift from the ABI the tests exercise through ctypes."""
    import importlib.util
    from pathlib import Path

    root = Path(__file__).resolve().parents[1]
    spec = importlib.util.spec_from_file_location("gen_ffi", root / "crates" / "decide-cuda" / "gen_ffi.py")
    gen = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(gen)
    text = (root / "crates" / "decide-cuda" / "src" / "ffi.rs").read_text()
    assert text == gen.render(), "run `python crates/decide-cuda/gen_ffi.py` after changing include/decide_cuda.h"
    declared = set(_lib.header_prototypes())
    assert all(f"pub fn {name}(" in text for name in declared) and len(declared) >= 50


def test_stale_library_is_refused(monkeypatch):
    """The stale-binary guard (the reference's source hash, crates/decide-metal/src/source_hash.rs): the library carries the
    hash of the sources it was built from; when the sources beside it hash differently, loading fails until it is rebuilt."""
    from decide_b200 import build

    lib = _lib.load()
    assert lib.dc_source_hash().decode() == build.source_hash() and len(build.source_hash()) == 16
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(build, "source_hash", lambda: "0" * 16)
    with pytest.raises(RuntimeError, match="built from other sources"):
        _lib.load()
    monkeypatch.setenv("DECIDE_ALLOW_STALE_LIBRARY", "1")
    assert _lib.load() is not None
