"""pytest configuration: the `gpu` marker and shared fixtures.

`-m "not gpu"` runs on a CPU-only machine (oracle vs golden vectors, host logic, ABI surface);
`-m gpu` runs the parity tests proper through the C ABI on a B200.
"""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100a) GPU; run with -m gpu")


@pytest.fixture(scope="session")
def dev():
    import torch

    if not torch.cuda.is_available():
        pytest.fail("a gpu-marked test was selected but no CUDA device is visible")
    from decide_b200.kernels import Device

    d = Device(0)
    yield d
    d.close()


@pytest.fixture(scope="session")
def k(dev):
    from decide_b200.kernels import Kernels

    return Kernels(dev)


@pytest.fixture(params=["f16", "bf16"])
def act(request, dev):
    """Runs the test once per activation storage type; yields the torch dtype of activation buffers."""
    from decide_b200.kernels import Act

    dev.set_activation_dtype(Act.F16 if request.param == "f16" else Act.BF16)
    yield dev.act_torch
    dev.set_activation_dtype(Act.F16)
