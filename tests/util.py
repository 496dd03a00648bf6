"""Helpers shared by the kernel tests, after the reference's crates/decide-engine/src/testutil.rs:
seeded inputs, inputs rounded through bf16 so the CPU reference sees what the GPU sees, and
assert_close(atol + rtol*|want|) that fails on NaN and reports how much of the tolerance was used."""
import numpy as np
import torch


def randn(seed: int, *shape, std: float = 1.0, mean: float = 0.0) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g, dtype=torch.float32) * std + mean


def uniform(seed: int, *shape, lo: float = 0.0, hi: float = 1.0) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    return torch.rand(*shape, generator=g, dtype=torch.float32) * (hi - lo) + lo


def bf16(x: torch.Tensor) -> torch.Tensor:
    """fp32 tensor -> bf16 tensor (round to nearest even)."""
    return x.to(torch.bfloat16)


def np32(x: torch.Tensor) -> np.ndarray:
    return x.detach().float().cpu().numpy()


def assert_close(got, want, atol: float, rtol: float, what: str = ""):
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, f"{what}: shape {got.shape} != {want.shape}"
    assert np.isfinite(got).all(), f"{what}: non-finite values in the result"
    tol = atol + rtol * np.abs(want)
    err = np.abs(got - want)
    used = float((err / tol).max()) if err.size else 0.0
    if used > 1.0:
        i = np.unravel_index(int(np.argmax(err / tol)), err.shape)
        raise AssertionError(
            f"{what}: max error {err.max():.3e}, {used * 100:.0f}% of tolerance at {i}: got {got[i]!r}, want {want[i]!r}")
    return used


def half_ulp(dtype) -> float:
    """Relative rounding step of a 16-bit activation type, with a little slack."""
    return 2 ** -8 if dtype == torch.bfloat16 else 2 ** -10
