"""Row kernels on the GPU (RMSNorm, embedding gather, row gathers, candidate-row head, gated
RMSNorm) against the restated cpu_ref functions. Outputs are bf16 (half-ulp 2^-9 relative) or fp32."""
import numpy as np
import pytest
import torch

from oracle import cpu_ref
from tests.util import assert_close, bf16, half_ulp, np32, randn

pytestmark = pytest.mark.gpu

H = 2560


@pytest.mark.parametrize("rows,h,add_one", [(1, 2560, True), (603, 2560, True), (77, 128, False), (9, 4096, True)])
def test_rmsnorm(k, rows, h, add_one, act):
    x = randn(1, rows, h)
    w = randn(2, h, std=0.02) if add_one else randn(2, h, std=0.02, mean=1.0)
    y = torch.empty(rows, h, dtype=act, device="cuda")
    k.norm.rmsnorm(None, x.cuda(), w.cuda(), y, None, rows, h, h, h, add_one)
    want = cpu_ref.rmsnorm(np32(x), np32(w), h, add_one)
    assert_close(np32(y), want, atol=1e-5, rtol=half_ulp(act), what="rmsnorm")


def test_rmsnorm_rowmap_and_strides(k):
    rows, h = 40, 256
    x = randn(3, 100, h + 4)
    w = randn(4, h, std=0.02)
    rowmap = torch.tensor(np.random.RandomState(0).permutation(100)[:rows].astype(np.int32))
    y = torch.full((rows, h + 8), 3.0, dtype=k.dev.act_torch, device="cuda")
    k.norm.rmsnorm(None, x.cuda(), w.cuda(), y, rowmap.cuda(), rows, h, h + 4, h + 8, True)
    want = cpu_ref.rmsnorm(np32(x)[rowmap.numpy(), :h], np32(w), h, True)
    assert_close(np32(y)[:, :h], want, atol=1e-5, rtol=2 ** -8, what="rmsnorm rowmap")
    assert (np32(y)[:, h:] == 3.0).all()


def test_rmsnorm_by_hand(k):
    """The reference's known answer (cpu_ref.rs:204-211) scaled to the kernel's 4-wide vectors."""
    x = torch.tensor([[3.0, 4.0, 3.0, 4.0]])
    w = torch.ones(4)
    y = torch.empty(1, 4, dtype=k.dev.act_torch, device="cuda")
    k.norm.rmsnorm(None, x.cuda(), w.cuda(), y, None, 1, 4, 4, 4, True)
    want = np.array([[3.0, 4.0, 3.0, 4.0]]) * 2.0 / np.sqrt(12.5)
    assert_close(np32(y), want, atol=0, rtol=2 ** -8, what="rmsnorm KAT")


def test_embed(k):
    vocab, t = 5000, 333
    table = bf16(randn(5, vocab, H, std=0.02))
    ids = torch.randint(0, vocab, (t,), generator=torch.Generator().manual_seed(6), dtype=torch.int32)
    out = torch.empty(t, H, dtype=torch.float32, device="cuda")
    k.embed.embed(None, ids.cuda(), table.cuda(), out, t, H)
    assert torch.equal(out.cpu(), table[ids.long()].float())


def test_gathers(k):
    x = randn(7, 64, H)
    rowmap = torch.tensor([5, 5, 63, 0, 17], dtype=torch.int32)
    out = torch.empty(5, H, dtype=torch.float32, device="cuda")
    k.head.gather_rows_f32(None, x.cuda(), rowmap.cuda(), out, 5, H)
    assert torch.equal(out.cpu(), x[rowmap.long()])
    xb = bf16(x)
    outb = torch.empty(5, H, dtype=torch.bfloat16, device="cuda")
    k.head.gather_rows_bf16(None, xb.cuda(), rowmap.cuda(), outb, 5, H)
    assert torch.equal(outb.cpu(), xb[rowmap.long()])


@pytest.mark.parametrize("rows,max_cand", [(6, 16), (16, 62), (1, 1)])
def test_final_head(k, rows, max_cand):
    vocab = 3000
    table = bf16(randn(8, vocab, H, std=0.02))
    x = randn(9, rows, H, std=3.0)
    w = randn(10, H, std=0.02)
    g = torch.Generator().manual_seed(11)
    ncand = torch.randint(1, max_cand + 1, (rows,), generator=g, dtype=torch.int32)
    ncand[0] = max_cand
    cand = torch.randint(0, vocab, (rows, max_cand), generator=g, dtype=torch.int32)
    logits = torch.full((rows, max_cand), -77.0, dtype=torch.float32, device="cuda")
    k.head.final_head(None, x.cuda(), w.cuda(), table.cuda(), cand.cuda(), ncand.cuda(), logits, rows, H, max_cand)
    cands = [np32(table[cand[r, :ncand[r]].long()]) for r in range(rows)]
    want = cpu_ref.final_head(np32(x), np32(w), cands, H)
    got = np32(logits)
    for r in range(rows):
        n = int(ncand[r])
        assert_close(got[r, :n], want[r], atol=2e-5, rtol=1e-5, what=f"final_head row {r}")
        assert (got[r, n:] == -77.0).all(), "entries past ncand must not be written"


@pytest.mark.parametrize("t,nv", [(1, 16), (603, 16), (50, 32)])
def test_gated_rmsnorm_silu(k, t, nv, act):
    dv, ldz = 128, nv * 128 + 96
    o = randn(12, t, nv * dv, std=0.5)
    z = randn(13, t, ldz)
    w = randn(14, dv, std=0.02, mean=1.0)
    y = torch.empty(t, nv * dv, dtype=act, device="cuda")
    k.gnorm.gated_rmsnorm_silu(None, o.cuda(), z.cuda(), w.cuda(), y, t, ldz, nv)
    want = cpu_ref.gated_rmsnorm_silu(np32(o), np32(z), ldz, np32(w), t, nv, dv)
    assert_close(np32(y), want, atol=1e-5, rtol=half_ulp(act), what="gated_rmsnorm_silu")


def test_convert_bf16_to_f16_with_report(k):
    """The weight converter's rounding and its precision-loss counters (convert.rs:73-90)."""
    from decide_b200.kernels import ConvertReport

    x = randn(20, 4096, std=0.02)
    x[:8] = torch.tensor([0.0, 1e-5, -3e-6, 1e-9, 7e4, -1e30, 3e4, 6.2e-5])  # subnormal x2, flushed, overflow x2
    src = bf16(x)
    rep = ConvertReport()
    out = k.dev.convert_bf16_to_f16(src.clone().cuda(), rep)
    want = src.float().to(torch.float16)
    assert torch.equal(out.cpu(), want)
    mag = want.float().abs()
    finite_src = torch.isfinite(src.float())
    assert rep.values == 4096
    assert rep.f16_overflow == int((torch.isinf(want) & finite_src).sum())
    assert rep.f16_flushed_to_zero == int(((want == 0) & (src.float() != 0)).sum())
    assert rep.f16_subnormal == int(((mag > 0) & (mag < 2 ** -14)).sum())
    assert rep.f16_overflow == 2 and rep.f16_flushed_to_zero >= 1 and rep.f16_subnormal >= 2


@pytest.mark.parametrize("h", [2560, 512])
@pytest.mark.parametrize("add16", [False, True])
def test_add_rmsnorm(k, h, add16, act):
    """The partial-sum add fused with the RMSNorm that follows (a tensor-parallel shard's norm): x += add in fp32, bit for bit;
    then the norm of the sum. fp32 and 16-bit partial sums, the register-resident form (H = 2560) and the generic one."""
    rows = 37
    x = randn(81, rows, h)
    add = randn(82, rows, h, std=0.5)
    add_dev = add.to(act) if add16 else add
    w = randn(83, h, std=0.02)
    xd = x.cuda()
    y = torch.empty(rows, h, dtype=act, device="cuda")
    k.norm.add_rmsnorm(None, xd, add_dev.cuda(), w.cuda(), y, rows, h)
    want_x = np32(x) + np32(add_dev.float())
    assert np.array_equal(np32(xd), want_x)
    want = cpu_ref.rmsnorm(want_x, np32(w), h, True)
    assert_close(np32(y), want, atol=1e-3 if act == torch.float16 else 8e-3, rtol=half_ulp(act), what="add_rmsnorm")
    x2 = x.cuda()
    k.norm.add_rmsnorm(None, x2, add_dev.cuda(), None, None, rows, h)      # only the add
    assert np.array_equal(np32(x2), want_x)
