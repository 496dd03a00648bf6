"""The allocation-free weight conversion, dc_convert_bf16_to_f16_noalloc, through the C ABI.

It serves hosts that cannot call cudaMalloc when they convert a checkpoint: a server swapping
weights in next to a stream that is answering requests (an allocation stalls the whole device), or a
process whose device memory already belongs to one arena. Its counters sit in a static array inside
the library instead of the context's workspace, so the checks here are: same fp16 bits and the same
precision-loss report as the ordinary entry point, on two calls in a row (the second must not see
the first call's counts), and a clear refusal beyond its per-call limit.

This file sorts last on purpose: a run that stops at the first failure has then already run every
other test. It passes alone in a fresh process as well as after the others.
"""
import ctypes

import pytest
import torch

from tests.util import randn

pytestmark = pytest.mark.gpu


def _inputs(seed):
    x = randn(seed, 70001, std=0.02)
    x[:6] = torch.tensor([1e-5, -3e-6, 1e-9, 7e4, -1e30, 6.2e-5]) * (1 + seed)
    return x.to(torch.bfloat16)


def test_noalloc_matches_the_allocating_entry_point_twice(dev):
    from decide_b200.kernels import ConvertReport

    lib = dev.lib
    stream = torch.cuda.current_stream().cuda_stream
    err = ctypes.create_string_buffer(256)
    for seed in (1, 2):  # two calls in a row, different data: the shared scratch must be cleared in between
        src = _inputs(seed)
        want_rep = ConvertReport()
        want = dev.convert_bf16_to_f16(src.clone().cuda(), want_rep)
        got_buf = src.clone().cuda()
        got_rep = ConvertReport()
        rc = lib.dc_convert_bf16_to_f16_noalloc(stream, got_buf.data_ptr(), got_buf.data_ptr(), got_buf.numel(), ctypes.byref(got_rep), err, len(err))
        assert rc == 0, err.value.decode()
        assert torch.equal(got_buf.view(torch.float16), want)  # bit-exact: integer/byte work
        assert got_rep.as_dict() == want_rep.as_dict()
        assert got_rep.f16_overflow == 2 and got_rep.f16_subnormal >= 1
    # out of place, no report, empty input
    src = _inputs(3).cuda()
    dst = torch.empty_like(src)
    assert lib.dc_convert_bf16_to_f16_noalloc(stream, src.data_ptr(), dst.data_ptr(), src.numel(), None, err, len(err)) == 0
    assert torch.equal(dst.view(torch.float16), src.float().to(torch.float16))
    assert lib.dc_convert_bf16_to_f16_noalloc(stream, src.data_ptr(), dst.data_ptr(), 0, None, err, len(err)) == 0


def test_noalloc_leaves_free_memory_alone(dev):
    """The property in the name: once the entry point has run on the device (the first call makes the driver
    load the kernel image), further calls take no device memory."""
    lib = dev.lib
    stream = torch.cuda.current_stream().cuda_stream
    err = ctypes.create_string_buffer(256)
    buf = _inputs(4).cuda()
    assert lib.dc_convert_bf16_to_f16_noalloc(stream, buf.data_ptr(), buf.data_ptr(), 0, None, err, len(err)) == 0   # warm
    assert lib.dc_convert_bf16_to_f16_noalloc(stream, buf.data_ptr(), buf.data_ptr(), buf.numel(), None, err, len(err)) == 0
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    for _ in range(3):
        src = buf   # no torch allocation inside the measured region
        assert lib.dc_convert_bf16_to_f16_noalloc(stream, src.data_ptr(), src.data_ptr(), src.numel(), None, err, len(err)) == 0
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before


def test_noalloc_refuses_more_than_its_limit(dev):
    lib = dev.lib
    err = ctypes.create_string_buffer(256)
    buf = torch.zeros(16, dtype=torch.bfloat16, device="cuda")
    rc = lib.dc_convert_bf16_to_f16_noalloc(torch.cuda.current_stream().cuda_stream, buf.data_ptr(), buf.data_ptr(), (1 << 32) + 1, None, err, len(err))
    assert rc == 1 and b"2^32" in err.value
    rc = lib.dc_convert_bf16_to_f16_noalloc(torch.cuda.current_stream().cuda_stream, None, buf.data_ptr(), 4, None, err, len(err))
    assert rc == 1 and b"null" in err.value
