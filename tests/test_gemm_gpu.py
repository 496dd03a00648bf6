"""GEMM parity on the GPU, through the C ABI, against the restated cpu_ref::gemm_nt +
swiglu_interleaved (oracle/cpu_ref.py). Inputs are seeded, rounded to bf16 once, and shared
bit-for-bit by both sides. X and W are stored in the context's 16-bit type (fp16 by default, bf16
also run). Tolerances: fp32 outputs atol 2e-4 + rtol 2e-5 (fp32 accumulation of
up to 9728 bf16 products of magnitude ~0.02); bf16 outputs add bf16's half-ulp, rtol 2^-8."""
import numpy as np
import pytest
import torch

from oracle import cpu_ref
from tests.util import assert_close, bf16, half_ulp, np32, randn

pytestmark = pytest.mark.gpu

F32_TOL = dict(atol=2e-4, rtol=2e-5)
BF16_TOL = dict(atol=2e-3, rtol=2 ** -8)


def _operands(seed, m, n, k, ldx=None, ldw=None, act=torch.float16):
    """X and W in the context's 16-bit type, rounded once and shared with the oracle."""
    ldx, ldw = ldx or k, ldw or k
    x = torch.zeros(m, ldx, dtype=act)
    w = torch.zeros(n, ldw, dtype=act)
    x[:, :k] = randn(seed, m, k).to(act)
    w[:, :k] = randn(seed + 1, n, k, std=0.02).to(act)
    return x, w


def _want(x, w, m, n, k, epi, y0=None, block=16):
    acc = cpu_ref.gemm_nt(np32(x[:, :k]), np32(w[:, :k]), m, n, k)
    if epi == 3:
        return cpu_ref.swiglu_interleaved(acc, m, n, block)
    if epi == 2:
        return acc + y0
    return acc


def _run(k, x, w, m, n, kk, epi, ldy=None, y0=None, bn=None, block=16):
    from decide_b200.kernels import Epilogue

    n_out = n // 2 if epi == 3 else n
    ldy = ldy or n_out
    dt = torch.float32 if epi in (0, 2) else k.dev.act_torch
    if y0 is not None:
        y = torch.zeros(m, ldy, dtype=dt)
        y[:, :n_out] = torch.from_numpy(y0)
        y = y.cuda()
    else:
        y = torch.full((m, ldy), 7.0, dtype=dt, device="cuda")  # canary: columns past n_out must stay 7
    xd, wd = x.cuda(), w.cuda()
    if bn is None:
        k.gemm.gemm(None, xd, wd, y, m, n, kk, x.shape[1], w.shape[1], ldy, Epilogue(epi), block)
    else:
        k.gemm.gemm_tile(None, xd, wd, y, m, n, kk, x.shape[1], w.shape[1], ldy, Epilogue(epi), bn)
    k.dev.check_status()
    out = np32(y)
    if ldy > n_out and y0 is None:
        assert (out[:, n_out:] == 7.0).all(), "the kernel wrote past the output columns"
    return out[:, :n_out]


@pytest.mark.parametrize("bn", [128, 192, 224, 256])
@pytest.mark.parametrize("m,n,kk", [(128, 256, 64), (128, 256, 256), (1, 32, 32), (37, 96, 160), (276, 512, 2560),
                                    (300, 8224, 512), (603, 2560, 1024)])
def test_fast_store_f32_shapes(k, m, n, kk, bn, act):
    """One tile / one k-block up to ragged M, N and K tails (TMA zero fill + masked stores)."""
    x, w = _operands(10 + m, m, n, kk, act=act)
    got = _run(k, x, w, m, n, kk, 0, bn=bn)
    assert_close(got, _want(x, w, m, n, kk, 0), what=f"StoreF32 {m}x{n}x{kk} bn{bn}", **F32_TOL)


@pytest.mark.parametrize("epi", [0, 1, 2, 3])
@pytest.mark.parametrize("bn", [128, 192, 224, 256])
def test_fast_epilogues(k, epi, bn, act):
    m, n, kk = 276, 1024, 2560
    x, w = _operands(3, m, n, kk, act=act)
    y0 = np32(randn(5, m, n)) if epi == 2 else None
    got = _run(k, x, w, m, n, kk, epi, y0=y0, bn=bn)
    tol = F32_TOL if epi in (0, 2) else dict(atol=2e-3, rtol=half_ulp(act))
    assert_close(got, _want(x, w, m, n, kk, epi, y0), what=f"epilogue {epi} bn{bn}", **tol)


def test_fast_strides_and_slices(k):
    """Row strides wider than K / N, and a row slice of W by offset (gemm.rs:126-130)."""
    from decide_b200.kernels import Epilogue

    m, n, kk = 200, 640, 320
    x, w = _operands(21, m, n, kk, ldx=kk + 64, ldw=kk + 8)
    got = _run(k, x, w, m, n, kk, 0, ldy=n + 12)
    assert_close(got, _want(x, w, m, n, kk, 0), what="strided", **F32_TOL)
    # rows 128..384 of W as a slice
    xd, wd = x.cuda(), w.cuda()
    y = torch.zeros(m, 256, dtype=torch.float32, device="cuda")
    k.gemm.gemm(None, xd, (wd, 128 * w.shape[1] * 2), y, m, 256, kk, x.shape[1], w.shape[1], 256, Epilogue.StoreF32)
    k.dev.check_status()
    want = cpu_ref.gemm_nt(np32(x[:, :kk]), np32(w[128:384, :kk]), m, 256, kk)
    assert_close(np32(y), want, what="W row slice", **F32_TOL)


def test_config0_gate_up_swiglu(k):
    """BASELINE config 0: X[276x2560] ~N(0,1), W_gate_up[19456x2560] ~N(0,0.02) -> SiLU(gate)*up [276x9728]."""
    m, n, kk = 276, 19456, 2560
    x, w = _operands(0, m, n, kk)
    got = _run(k, x, w, m, n, kk, 3)
    assert_close(got, _want(x, w, m, n, kk, 3), what="config 0", **BF16_TOL)


# Shapes whose last, partial wave of tiles is cut along K (the down projection of the benchmark at 603 and
# 2,307 rows; the same with an N tail; a forced 128-wide tile). (m, n, k, forced tile width or None)
SPLIT_SHAPES = [(603, 2560, 9728, None), (2307, 2560, 9728, None), (603, 2592, 9728, None), (300, 2560, 9728, 128)]


@pytest.mark.parametrize("m,n,kk,bn", SPLIT_SHAPES)
def test_k_split_tail_wave(k, m, n, kk, bn, act):
    """The tail-wave K split: parts park fp32 partials in the context's workspace and the last epilogue warp to
    arrive sums them in part order. Every epilogue, both 16-bit types, M and N tails; each case runs twice and
    the two results must be bit-identical (arrival order must not matter, the arrival counters must be back at
    zero). The plan is asserted first so that this test cannot silently stop covering the split path."""
    from decide_b200.kernels import Epilogue

    splits = {epi: k.gemm.plan_for(m, n, kk, Epilogue(epi), bn or 0)[1] for epi in (0, 1, 2, 3)}
    assert min(splits.values()) >= 2, f"plan for {m}x{n}x{kk} no longer splits the tail wave for every epilogue ({splits}): pick another shape"
    x, w = _operands(50 + m + n, m, n, kk, act=act)
    acc = cpu_ref.gemm_nt(np32(x), np32(w), m, n, kk)
    y0 = np32(randn(51, m, n))
    for epi in (0, 1, 2, 3):
        want = cpu_ref.swiglu_interleaved(acc, m, n, 16) if epi == 3 else (acc + y0 if epi == 2 else acc)
        tol = F32_TOL if epi in (0, 2) else dict(atol=2e-3, rtol=half_ulp(act))
        first = _run(k, x, w, m, n, kk, epi, y0=y0 if epi == 2 else None, bn=bn)
        assert_close(first, want, what=f"split {splits[epi]} epilogue {epi} {m}x{n}x{kk}", **tol)
        again = _run(k, x, w, m, n, kk, epi, y0=y0 if epi == 2 else None, bn=bn)
        assert np.array_equal(first, again), f"epilogue {epi}: two runs of a K-split GEMM differ"


def test_k_split_full_batch_tail_rows(k):
    """The benchmark's down projection at its full batch (38,592 rows): 3,020 tiles = 20 whole waves + 60 tail
    tiles cut in two. Checked on the rows of the tail tiles (the last requests of the batch) and a band of whole-tile rows."""
    from decide_b200.kernels import Epilogue

    m, n, kk = 38592, 2560, 9728
    bn, split = k.gemm.plan_k(m, n, kk)
    assert split >= 2, f"plan for {m}x{n}x{kk} no longer splits the tail wave"
    act = k.dev.act_torch
    g = torch.Generator(device="cuda").manual_seed(7)
    x = torch.randn(m, kk, generator=g, device="cuda").to(act)
    w = (torch.randn(n, kk, generator=g, device="cuda") * 0.02).to(act)
    y = torch.randn(m, n, generator=g, device="cuda")
    y0 = y.clone()
    k.gemm.gemm(None, x, w, y, m, n, kk, kk, kk, n, Epilogue.AddF32)
    k.dev.check_status()
    for lo, hi in ((0, 256), (m - 1024, m)):
        acc = cpu_ref.gemm_nt(np32(x[lo:hi]), np32(w), hi - lo, n, kk)
        assert_close(np32(y[lo:hi]), acc + np32(y0[lo:hi]), what=f"rows {lo}..{hi}", **F32_TOL)


@pytest.mark.parametrize("m", [1, 3, 6, 8, 9, 16])
@pytest.mark.parametrize("n,kk,epi", [(19456, 2560, 3), (2560, 9728, 2), (8224, 2560, 0), (2560, 2048, 1), (10240, 2560, 0),
                                      (32, 32, 0), (96, 160, 2), (64, 64, 3), (2560, 4096, 0)])
def test_small_m_streaming_gemm(k, m, n, kk, epi, act):
    """M <= 16 (the answer rows of the pruned last layer) runs the weight-streaming kernel (the reference's
    gemm_nt_small): every projection shape of the model, all four epilogues, every K split (1, 2, 4, 8), row counts
    on both sides of the MMA's 8-row halves, strided outputs with a canary."""
    if m not in (3, 16) and n * kk > 2 ** 22 and (n, kk) != (2560, 9728):
        pytest.skip("the large shapes run at M = 3 and 16 (and the down projection at every M)")
    x, w = _operands(70 + m + n, m, n, kk, act=act)
    y0 = np32(randn(71, m, n)) if epi == 2 else None
    n_out = n // 2 if epi == 3 else n
    got = _run(k, x, w, m, n, kk, epi, y0=y0, ldy=n_out + (0 if epi == 2 else 8))
    tol = F32_TOL if epi in (0, 2) else dict(atol=2e-3, rtol=half_ulp(act))
    assert_close(got, _want(x, w, m, n, kk, epi, y0), what=f"small-M {m}x{n}x{kk} epilogue {epi}", **tol)
    # and it agrees with the tcgen05 kernel on the same operands to fp32 summation order
    big = _run(k, x, w, m, n, kk, epi, y0=y0, bn=256)
    assert_close(got, big, what="small-M vs tcgen05", **(dict(atol=1e-4, rtol=1e-5) if epi in (0, 2) else dict(atol=2e-3, rtol=2 * half_ulp(act))))


@pytest.mark.parametrize("epi", [0, 1, 2, 3])
@pytest.mark.parametrize("block", [16, 32])
def test_baseline_kernel(k, epi, block, act):
    """The bisecting kernel (DECIDE_GEMM=baseline) against the same oracle, incl. other SwiGLU blocks."""
    from decide_b200.kernels import Family, Impl

    if epi != 3 and block != 16:
        pytest.skip("block only matters for SwiGLU")
    m, n, kk = 70, 192, 96
    x, w = _operands(40, m, n, kk, act=act)
    y0 = np32(randn(41, m, n)) if epi == 2 else None
    k.dev.set_impl(Family.Gemm, Impl.Baseline)
    try:
        got = _run(k, x, w, m, n, kk, epi, y0=y0, block=block)
    finally:
        k.dev.set_impl(Family.Gemm, Impl.Fast)
    tol = F32_TOL if epi in (0, 2) else BF16_TOL
    assert_close(got, _want(x, w, m, n, kk, epi, y0, block), what=f"baseline epilogue {epi}", **tol)


def test_fast_equals_baseline_bitwise_when_exact(k):
    """Small integers: every product and partial sum is exact in fp32, so fast and baseline must agree bit for bit."""
    from decide_b200.kernels import Epilogue, Family, Impl

    m, n, kk = 130, 288, 192
    g = torch.Generator().manual_seed(9)
    x = torch.randint(-4, 5, (m, kk), generator=g).to(k.dev.act_torch).cuda()
    w = torch.randint(-4, 5, (n, kk), generator=g).to(k.dev.act_torch).cuda()
    outs = []
    for impl in (Impl.Fast, Impl.Baseline):
        k.dev.set_impl(Family.Gemm, impl)
        y = torch.zeros(m, n, dtype=torch.float32, device="cuda")
        k.gemm.gemm(None, x, w, y, m, n, kk, kk, kk, n, Epilogue.StoreF32)
        k.dev.check_status()
        outs.append(y.cpu())
    k.dev.set_impl(Family.Gemm, Impl.Fast)
    assert torch.equal(outs[0], outs[1])
    assert torch.equal(outs[0], (x.float().cpu() @ w.float().cpu().T))


def test_contract_violations_are_errors(k):
    """What the reference asserts (gemm.rs:140-144, 159-163) comes back as DC_INVALID_ARG, nothing is launched."""
    from decide_b200.kernels import Epilogue, KernelError

    x = torch.zeros(4, 64, dtype=k.dev.act_torch, device="cuda")
    w = torch.zeros(64, 64, dtype=k.dev.act_torch, device="cuda")
    y = torch.zeros(4, 64, dtype=torch.float32, device="cuda")
    before = k.dev.launches
    for args in [(4, 48, 64, 64, 64, 64), (4, 64, 48, 64, 64, 64), (0, 64, 64, 64, 64, 64), (4, 64, 64, 32, 64, 64),
                 (4, 64, 64, 64, 64, 32), (4, 64, 64, 68, 64, 64)]:
        with pytest.raises(KernelError) as e:
            k.gemm.gemm(None, x, w, y, *args, Epilogue.StoreF32)
        assert e.value.code == 1
    with pytest.raises(KernelError) as e:
        k.gemm.gemm(None, x, w, y, 4, 64, 64, 64, 64, 32, Epilogue.SwigluBF16, 32)
    assert e.value.code in (1, 3)
    assert k.dev.launches == before


def test_a_wait_that_runs_out_is_reported_and_the_context_survives(k):
    """Failure detection without a fault: a kernel whose only wait is on a barrier nothing arrives at gives up at the
    library's limit, raises the device status word and returns; dc_check_status reports DC_TIMEOUT once (with the wait's
    id), clears the word, and the same context then runs a GEMM correctly."""
    from decide_b200.kernels import Epilogue, KernelError

    k.dev.check_status()                       # clean to start with
    k.dev.selftest_wait_timeout()
    with pytest.raises(KernelError) as err:
        k.dev.check_status()
    assert err.value.code == 4 and "wait id 99" in str(err.value)
    k.dev.check_status()                       # latched once, cleared by the report
    m, n, kk = 130, 256, 128
    x = randn(5, m, kk).to(k.dev.act_torch).cuda()
    w = randn(6, n, kk, std=0.05).to(k.dev.act_torch).cuda()
    y = torch.empty(m, n, device="cuda")
    k.gemm.gemm(None, x, w, y, m, n, kk, kk, kk, n, Epilogue.StoreF32)
    k.dev.check_status()
    want = x.float() @ w.float().T
    assert torch.allclose(y, want, atol=1e-2, rtol=1e-2)
