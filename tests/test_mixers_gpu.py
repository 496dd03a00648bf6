"""The attention-side and Gated-DeltaNet-side kernels on the GPU against the restated cpu_ref
functions: head norm + RoPE, K/V cache write, causal GQA attention (fast and baseline, gated and
un-gated, packed sequences), conv + SiLU + L2 norm, conv state update, the gated delta rule (state
carry across chunks, packed sequences, the reference's by-hand known answer)."""
import math

import numpy as np
import pytest
import torch

from oracle import cpu_ref
from tests.util import assert_close, bf16, half_ulp, np32, randn, uniform

pytestmark = pytest.mark.gpu


def _u32(x):
    return torch.as_tensor(np.asarray(x, dtype=np.int32)).cuda()


# ------------------------------------------------------------------ rope
@pytest.mark.parametrize("hd,rot,theta,nq", [(128, 128, 1e6, 32), (256, 64, 1e7, 16), (128, 32, 1e6, 4)])
def test_q_norm_rope(k, hd, rot, theta, nq, act):
    rows, ldq = 50, nq * hd + 64
    pq = randn(1, rows, ldq)
    w = randn(2, hd, std=0.02)
    qpos = np.random.RandomState(3).randint(0, 8192, rows)
    qpos[0], qpos[1] = 0, 8191
    inv_freq = torch.from_numpy(cpu_ref.inv_freq(rot, theta))
    qo = torch.empty(rows, nq, hd, dtype=act, device="cuda")
    k.rope.q_norm_rope(None, pq.cuda(), w.cuda(), inv_freq.cuda(), _u32(qpos), qo, rows, ldq, nq, hd, rot)
    seg = np32(pq)[:, :nq * hd].reshape(rows, nq, hd)
    want = cpu_ref.head_norm_rope(seg, np32(w), qpos[:, None].repeat(nq, 1), rot, theta)
    # fp32 angles up to 8191 rad: sin/cos of the same fp32 angle, so only bf16 rounding remains
    assert_close(np32(qo), want, atol=2e-3 if act == torch.bfloat16 else 3e-4, rtol=half_ulp(act), what="q_norm_rope")


@pytest.mark.parametrize("packed", [False, True])
def test_kv_norm_rope(k, packed):
    hd, rot, theta, nkv = 128, 128, 1e6, 8
    rows, ld, kcol, vcol, pos0, cache_rows = 37, 6144, 4096, 5120, 11, 64
    p = randn(4, rows, ld)
    w = randn(5, hd, std=0.02)
    inv_freq = torch.from_numpy(cpu_ref.inv_freq(rot, theta))
    act = k.dev.act_torch
    kc = torch.full((cache_rows, nkv, hd), 9.0, dtype=act, device="cuda")
    vc = torch.full((cache_rows, nkv, hd), 9.0, dtype=act, device="cuda")
    if packed:
        pos = np.concatenate([np.arange(20), np.arange(17)])
        k.rope.kv_norm_rope(None, p.cuda(), w.cuda(), inv_freq.cuda(), kc, vc, rows, ld, kcol, vcol, 0, cache_rows, nkv, hd, rot,
                            pos=_u32(pos))
        dst = np.arange(rows)
    else:
        pos = pos0 + np.arange(rows)
        k.rope.kv_norm_rope(None, p.cuda(), w.cuda(), inv_freq.cuda(), kc, vc, rows, ld, kcol, vcol, pos0, cache_rows, nkv, hd, rot)
        dst = pos
    kseg = np32(p)[:, kcol:kcol + nkv * hd].reshape(rows, nkv, hd)
    want_k = cpu_ref.head_norm_rope(kseg, np32(w), pos[:, None].repeat(nkv, 1), rot, theta)
    assert_close(np32(kc)[dst], want_k, atol=2e-3, rtol=2 ** -8, what="k cache")
    want_v = np32(p[:, vcol:vcol + nkv * hd].to(act)).reshape(rows, nkv, hd)
    assert np.array_equal(np32(vc)[dst], want_v)
    untouched = np.setdiff1d(np.arange(cache_rows), dst)
    assert (np32(kc)[untouched] == 9.0).all() and (np32(vc)[untouched] == 9.0).all()


def test_kv_cache_overrun_is_refused(k):
    from decide_b200.kernels import KernelError

    z = torch.zeros(8, 2048, device="cuda")
    c = torch.zeros(8, 8, 128, dtype=k.dev.act_torch, device="cuda")
    with pytest.raises(KernelError):
        k.rope.kv_norm_rope(None, z, z, z, c, c, 8, 2048, 0, 1024, 1, 8, 8, 128, 128)


# ------------------------------------------------------------- attention
def _attn_case(seed, rows, nq, nkv, hd, gated, qpos=None, npos=None, act=torch.float16):
    npos = npos or rows
    q = randn(seed, rows, nq, hd).to(act)
    kc = randn(seed + 1, npos, nkv, hd).to(act)
    vc = randn(seed + 2, npos, nkv, hd).to(act)
    gate = randn(seed + 3, rows, nq * hd + 32) if gated else None
    qpos = np.arange(rows) if qpos is None else qpos
    want = cpu_ref.attention(np32(q), qpos, np32(kc), np32(vc), np32(gate)[:, :nq * hd] if gated else None, nq, nkv, hd)
    return q, kc, vc, gate, qpos, want


@pytest.mark.parametrize("impl", ["fast", "baseline"])
@pytest.mark.parametrize("rows,gated", [(1, True), (64, False), (65, True), (300, True), (603, False)])
def test_attention_single_sequence(k, impl, rows, gated, act):
    from decide_b200.kernels import Family, Impl

    nq, nkv, hd = 8, 2, 128
    q, kc, vc, gate, qpos, want = _attn_case(10 + rows, rows, nq, nkv, hd, gated, act=act)
    y = torch.empty(rows, nq * hd, dtype=act, device="cuda")
    k.dev.set_impl(Family.Attn, Impl.Baseline if impl == "baseline" else Impl.Fast)
    try:
        k.attn.attention(None, q.cuda(), kc.cuda(), vc.cuda(), gate.cuda() if gated else None, _u32(qpos), y, rows,
                         gate.shape[1] if gated else 0, nq, nkv, hd)
        k.dev.check_status()
    finally:
        k.dev.set_impl(Family.Attn, Impl.Fast)
    # P is rounded to the activation type before PV in the fast kernel (as the reference rounds to fp16): atol covers it
    assert_close(np32(y), want, atol=6e-3 if act == torch.bfloat16 else 1e-3, rtol=2 * half_ulp(act), what=f"attention {impl} rows={rows}")


def test_attention_scattered_query_positions(k):
    """Query rows at arbitrary positions of a longer cache (the pruned-last-layer form, forward.rs:1176-1178)."""
    nq, nkv, hd, npos = 4, 1, 128, 500
    qpos = np.array([499, 3, 250, 0, 77, 77, 128, 64, 63])
    q, kc, vc, gate, qpos, want = _attn_case(40, len(qpos), nq, nkv, hd, True, qpos=qpos, npos=npos)
    y = torch.empty(len(qpos), nq * hd, dtype=k.dev.act_torch, device="cuda")
    k.attn.attention(None, q.cuda(), kc.cuda(), vc.cuda(), gate.cuda(), _u32(qpos), y, len(qpos), gate.shape[1], nq, nkv, hd)
    assert_close(np32(y), want, atol=6e-3, rtol=2 ** -7, what="attention scattered")


@pytest.mark.parametrize("rows,c0,gated", [(100, 400, True), (64, 0, False), (300, 1000, True), (129, 127, False), (63, 200, True)])
def test_attention_chunk_continuing_a_cache(k, rows, c0, gated, act):
    """A chunk of one request: rows at positions c0 .. c0 + rows over cache rows 0 .. c0 + rows (chunked prefill, the
    snapshot and state-cache routes, forward.rs:919-942). With the cache length given, a chunk of 64 rows or more runs on
    the tcgen05 kernel (63 rows: the mma.sync kernel). The cache buffers are longer than the rows in use and hold NaN
    past them: nothing there may be read."""
    nq, nkv, hd = 8, 2, 128
    kv_len = c0 + rows
    qpos = c0 + np.arange(rows)
    q, kc, vc, gate, qpos, want = _attn_case(70 + rows, rows, nq, nkv, hd, gated, qpos=qpos, npos=kv_len, act=act)
    pad = torch.full((77, nkv, hd), float("nan"), dtype=act)
    y = torch.full((rows + 1, nq * hd), 5.0, dtype=act, device="cuda")
    k.attn.attention(None, q.cuda(), torch.cat([kc, pad]).cuda(), torch.cat([vc, pad]).cuda(), gate.cuda() if gated else None, _u32(qpos), y, rows,
                     gate.shape[1] if gated else 0, nq, nkv, hd, max_len=kv_len)
    k.dev.check_status()
    assert_close(np32(y[:rows]), want, atol=6e-3 if act == torch.bfloat16 else 1e-3, rtol=2 * half_ulp(act), what=f"attention chunk rows={rows} c0={c0}")
    assert (np32(y[rows]) == 5.0).all()


def test_attention_reports_a_position_past_the_given_cache_length(k):
    """A caller that gives the cache length promises every position is below it; the kernel reads nothing past the length
    and the next status check reports the broken promise as an argument error, not as a result."""
    from decide_b200.kernels import KernelError

    nq, nkv, hd, rows = 8, 2, 128, 64
    q, kc, vc, _, _, _ = _attn_case(90, rows, nq, nkv, hd, False, qpos=np.arange(rows), npos=200, act=k.dev.act_torch)
    y = torch.empty(rows, nq * hd, dtype=k.dev.act_torch, device="cuda")
    k.attn.attention(None, q.cuda(), kc.cuda(), vc.cuda(), None, _u32(100 + np.arange(rows)), y, rows, 0, nq, nkv, hd, max_len=150)
    with pytest.raises(KernelError, match="at or past the cache length"):
        k.dev.check_status()
    k.dev.check_status()   # the context stays usable


@pytest.mark.parametrize("repeat", [1, 20], ids=["few-rows-sliced-keys", "many-rows"])
@pytest.mark.parametrize("gated", [True, False])
def test_attention_rows_over_packed_caches(k, gated, act, repeat):
    """The pruned last layer's attention: a few answer rows of several requests, each attending the cache rows of its own
    request up to its position (1 key, a tile boundary, more than two tiles of 256), 4 query heads per kv head. With few rows
    the kernel cuts each row's keys into slices and joins them (9 rows x 2 kv heads: 17 slices, most of them empty for the
    short rows); with many rows (180 x 2 CTAs) every row is one slice."""
    nq, nkv, hd = 8, 2, 128
    lens = [603, 1, 257, 700]
    starts = np.concatenate([[0], np.cumsum(lens)])
    total = int(starts[-1])
    kc = randn(61, total, nkv, hd).to(act)
    vc = randn(62, total, nkv, hd).to(act)
    picks = [(0, 602), (0, 0), (0, 255), (0, 256), (1, 0), (2, 256), (3, 699), (3, 511), (3, 512)] * repeat   # (request, position)
    rows = len(picks)
    q = randn(63, rows, nq, hd).to(act)
    gate = randn(64, rows, nq * hd + 16) if gated else None
    qpos = np.array([p for _, p in picks])
    kv0 = np.array([starts[s] for s, _ in picks])
    y = torch.full((rows + 1, nq * hd), 5.0, dtype=act, device="cuda")
    k.attn.attention_rows(None, q.cuda(), kc.cuda(), vc.cuda(), gate.cuda() if gated else None, _u32(qpos), _u32(kv0), y, rows,
                          gate.shape[1] if gated else 0, nq, nkv, hd)
    k.dev.check_status()
    for i, (s, p) in enumerate(picks):
        lo, hi = int(starts[s]), int(starts[s + 1])
        want = cpu_ref.attention(np32(q[i:i + 1]), np.array([p]), np32(kc[lo:hi]), np32(vc[lo:hi]),
                                 np32(gate)[i:i + 1, :nq * hd] if gated else None, nq, nkv, hd)
        assert_close(np32(y[i:i + 1]), want, atol=2e-3 if act == torch.bfloat16 else 3e-4, rtol=half_ulp(act), what=f"attention_rows {picks[i]}")
    assert (np32(y[rows]) == 5.0).all()


@pytest.fixture(params=["fast", "fast-mma", "baseline"])
def attn_impl(request, k):
    """Packed-batch attention on the tcgen05 kernel (fast), the mma.sync flash kernel (fast-mma) and the warp-per-row baseline."""
    from decide_b200.kernels import Engine, Family, Impl

    k.dev.set_impl(Family.Attn, Impl.Baseline if request.param == "baseline" else Impl.Fast)
    k.dev.set_engine(Family.Attn, Engine.MmaSync if request.param == "fast-mma" else Engine.Tcgen05)
    yield request.param
    k.dev.set_impl(Family.Attn, Impl.Fast)
    k.dev.set_engine(Family.Attn, Engine.Tcgen05)
    k.dev.check_status()


def _packed_attention(k, seed, lens, nq, nkv, gated=True, k_growth=0.0):
    hd = 128
    starts = np.concatenate([[0], np.cumsum(lens)])
    total = int(starts[-1])
    q = randn(seed, total, nq, hd).to(k.dev.act_torch)
    kc = randn(seed + 1, total, nkv, hd)
    if k_growth:   # later cache rows score higher and higher: the running maximum keeps growing
        kc = kc * (1.0 + k_growth * torch.arange(total).float())[:, None, None]
    kc = kc.to(k.dev.act_torch)
    vc = randn(seed + 2, total, nkv, hd).to(k.dev.act_torch)
    gate = randn(seed + 3, total, nq * hd) if gated else None
    qpos = np.concatenate([np.arange(n) for n in lens])
    y = torch.empty(total, nq * hd, dtype=k.dev.act_torch, device="cuda")
    k.attn.attention(None, q.cuda(), kc.cuda(), vc.cuda(), gate.cuda() if gated else None, _u32(qpos), y, total, nq * hd if gated else 0, nq, nkv, hd,
                     seq_start=_u32(starts), n_seq=len(lens), max_len=max(lens))
    k.dev.check_status()
    got = np32(y)
    for s, n in enumerate(lens):
        a, b = starts[s], starts[s + 1]
        want = cpu_ref.attention(np32(q)[a:b], np.arange(n), np32(kc)[a:b], np32(vc)[a:b], np32(gate)[a:b] if gated else None, nq, nkv, hd)
        assert_close(got[a:b], want, atol=6e-3, rtol=2 ** -7, what=f"packed attention seq {s} (len {n})")


def test_attention_packed_sequences(k, attn_impl):
    _packed_attention(k, 50, [70, 1, 130, 64], 8, 2)


def test_attention_packed_long_and_ragged(k, attn_impl):
    """Several 128-row tiles per sequence, sequence starts that are not multiples of 8, an un-gated call."""
    _packed_attention(k, 60, [603, 3, 257, 128, 129, 5], 4, 1, gated=False)


def test_attention_packed_growing_scores(k, attn_impl):
    """Scores that grow along the cache force the running maximum (and the rescaling of the output accumulator) to move in every tile."""
    _packed_attention(k, 70, [400, 300], 4, 2, k_growth=0.02)


# ------------------------------------------------------------------ conv
@pytest.mark.parametrize("t,nk,nv,with_prev", [(1, 16, 16, True), (2, 16, 16, False), (100, 16, 16, True), (35, 16, 32, True)])
def test_conv_silu_l2(k, t, nk, nv, with_prev):
    conv_dim = (2 * nk + nv) * 128
    ldp = conv_dim + 2080
    p = randn(60, t, ldp)
    prev = randn(61, 3, conv_dim) if with_prev else None
    w = randn(62, conv_dim, 4, std=0.3)
    q = torch.empty(t, nk, 128, device="cuda")
    kk = torch.empty(t, nk, 128, device="cuda")
    v = torch.empty(t, nv, 128, device="cuda")
    k.conv.conv_silu_l2(None, p.cuda(), prev.cuda() if with_prev else None, w.cuda(), q, kk, v, t, ldp, nk, nv)
    wq, wk, wv = cpu_ref.conv_silu_l2(np32(p), ldp, t, np32(prev) if with_prev else np.zeros((3, conv_dim), np.float32),
                                     np32(w), nk, nv, 128, 128)
    assert_close(np32(q), wq, atol=2e-6, rtol=2e-5, what="conv q")
    assert_close(np32(kk), wk, atol=2e-6, rtol=2e-5, what="conv k")
    assert_close(np32(v), wv, atol=2e-6, rtol=2e-5, what="conv v")


def test_conv_packed_sequences_equal_separate_calls(k):
    nk = nv = 16
    conv_dim = 48 * 128
    lens = [5, 40, 1, 17]
    starts = np.concatenate([[0], np.cumsum(lens)])
    total = int(starts[-1])
    p = randn(63, total, conv_dim).cuda()
    w = randn(64, conv_dim, 4, std=0.3).cuda()
    outs = [torch.empty(total, 16, 128, device="cuda") for _ in range(3)]
    k.conv.conv_silu_l2(None, p, None, w, *outs, total, conv_dim, nk, nv, seq_start=_u32(starts), n_seq=len(lens), max_len=max(lens))
    for s, n in enumerate(lens):
        a = int(starts[s])
        ref = [torch.empty(n, 16, 128, device="cuda") for _ in range(3)]
        k.conv.conv_silu_l2(None, p[a:a + n], None, w, *ref, n, conv_dim, nk, nv)
        for got, want in zip(outs, ref):
            assert torch.equal(got[a:a + n], want)


@pytest.mark.parametrize("t", [1, 2, 3, 50])
def test_conv_state_update(k, t):
    conv_dim, ldp = 6144, 8224
    p = randn(65, t, ldp)
    prev = randn(66, 3, conv_dim)
    buf = prev.clone().cuda()
    k.conv.conv_state_update(None, p.cuda(), buf, buf, t, ldp, conv_dim)  # in place, as the engine does
    want = cpu_ref.conv_state_update(np32(p), ldp, t, np32(prev), conv_dim)
    assert np.array_equal(np32(buf), want)


# ----------------------------------------------------------------- delta
@pytest.fixture(params=["chunked", "chunked-mma", "sequential"])
def delta_impl(request, k):
    """Runs a delta-rule test on the chunk-64 tensor-core kernels (fast; serial kernel on tcgen05 or on
    mma.sync) and on the sequential kernel (baseline)."""
    from decide_b200.kernels import Engine, Family, Impl

    k.dev.set_impl(Family.Delta, Impl.Baseline if request.param == "sequential" else Impl.Fast)
    k.dev.set_engine(Family.Delta, Engine.MmaSync if request.param == "chunked-mma" else Engine.Tcgen05)
    yield "sequential" if request.param == "sequential" else "chunked"
    k.dev.set_impl(Family.Delta, Impl.Fast)
    k.dev.set_engine(Family.Delta, Engine.Tcgen05)
    k.dev.check_status()


# fp32 sequential kernel vs the f64-accumulating oracle: ~1e-6; chunked kernel with hi/lo split operands: ~1e-5
DELTA_TOL = dict(atol=6e-5, rtol=3e-4)

def _delta_inputs(seed, t, nk, nv):
    q = randn(seed, t, nk, 128)
    kk = randn(seed + 1, t, nk, 128)
    q = q / q.norm(dim=-1, keepdim=True) * 128 ** -0.5
    kk = kk / kk.norm(dim=-1, keepdim=True)
    v = randn(seed + 2, t, nv, 128)
    ldab = nv + 8
    a = randn(seed + 3, t, ldab)
    b = randn(seed + 4, t, ldab)
    a_log = uniform(seed + 5, nv, lo=0.0, hi=math.log(16.0))
    dt_bias = randn(seed + 6, nv, std=0.02, mean=1.0)
    return q, kk, v, a, b, ldab, a_log, dt_bias


def _delta_gpu(k, q, kk, v, a, b, ldab, a_log, dt_bias, state, t, nk, nv, write=True, **kw):
    o = torch.empty(q.shape[0], nv, 128, device="cuda")
    k.delta.gated_delta(None, q.cuda(), kk.cuda(), v.cuda(), a.cuda(), b.cuda(), a_log.cuda(), dt_bias.cuda(), state, state, o, t,
                        ldab, write, nk, nv, **kw)
    return o


@pytest.mark.parametrize("t,nk,nv", [(1, 16, 16), (17, 16, 16), (64, 16, 16), (130, 16, 16), (40, 16, 32), (603, 16, 16)])
def test_gated_delta_vs_sequential_reference(k, t, nk, nv, delta_impl):
    q, kk, v, a, b, ldab, a_log, dt_bias = _delta_inputs(70 + t, t, nk, nv)
    s0 = randn(80, nv, 128, 128, std=0.1)
    state = s0.clone().cuda()
    o = _delta_gpu(k, q, kk, v, a, b, ldab, a_log, dt_bias, state, t, nk, nv)
    ref_state = np32(s0).copy()
    want = cpu_ref.gated_delta(np32(q), np32(kk), np32(v), np32(a), np32(b), ldab, np32(a_log), np32(dt_bias), ref_state, t, nk, nv, 128, 128)
    assert_close(np32(o), want, what="delta o", **DELTA_TOL)
    assert_close(np32(state), ref_state, what="delta state", **DELTA_TOL)


def test_gated_delta_by_hand(k, delta_impl):
    """The reference's known answer (cpu_ref.rs:222-236): one step, beta = 1, g = 1 -> o = v, S = k delta^T."""
    nk = nv = 16
    kk = torch.zeros(1, nk, 128)
    kk[0, :, 0] = 1.0
    v = torch.zeros(1, nv, 128)
    v[0, 0, 5] = 3.0
    a, b = torch.zeros(1, nv), torch.full((1, nv), 50.0)
    a_log = torch.full((nv,), -float("inf"))
    state = torch.zeros(nv, 128, 128, device="cuda")
    o = _delta_gpu(k, kk.clone(), kk, v, a, b, nv, a_log, torch.zeros(nv), state, 1, nk, nv)
    assert abs(o[0, 0, 5].item() - 3.0) < 1e-5
    assert abs(state[0, 5, 0].item() - 3.0) < 1e-5
    assert o.abs().sum().item() == pytest.approx(3.0, abs=1e-4)


def test_gated_delta_chunk_continuation_is_exact(k, delta_impl):
    """Whole sequence vs the same rows in two calls carrying the state (the engine's chunk continuation,
    forward.rs:1214-1234): fp32 through memory, so bit-identical. The chunked kernel regroups tokens by
    64, so for it the cut must fall on a chunk boundary to be bit-identical."""
    t, nk, nv = 150, 16, 16
    q, kk, v, a, b, ldab, a_log, dt_bias = _delta_inputs(90, t, nk, nv)
    s_whole = torch.zeros(nv, 128, 128, device="cuda")
    o_whole = _delta_gpu(k, q, kk, v, a, b, ldab, a_log, dt_bias, s_whole, t, nk, nv)
    s_split = torch.zeros(nv, 128, 128, device="cuda")
    cut = 64 if delta_impl == "chunked" else 33
    o1 = _delta_gpu(k, q[:cut], kk[:cut], v[:cut], a[:cut], b[:cut], ldab, a_log, dt_bias, s_split, cut, nk, nv)
    o2 = _delta_gpu(k, q[cut:], kk[cut:], v[cut:], a[cut:], b[cut:], ldab, a_log, dt_bias, s_split, t - cut, nk, nv)
    assert torch.equal(torch.cat([o1, o2]), o_whole)
    assert torch.equal(s_split, s_whole)


def test_gated_delta_write_state_false_leaves_state(k, delta_impl):
    t, nk, nv = 10, 16, 16
    q, kk, v, a, b, ldab, a_log, dt_bias = _delta_inputs(95, t, nk, nv)
    state = torch.full((nv, 128, 128), 0.25, device="cuda")
    _delta_gpu(k, q, kk, v, a, b, ldab, a_log, dt_bias, state, t, nk, nv, write=False)
    assert (state == 0.25).all()


def test_gated_delta_packed_sequences(k, delta_impl):
    nk = nv = 16
    lens = [20, 1, 145, 64]
    starts = np.concatenate([[0], np.cumsum(lens)])
    total = int(starts[-1])
    q, kk, v, a, b, ldab, a_log, dt_bias = _delta_inputs(97, total, nk, nv)
    states = torch.zeros(len(lens), nv, 128, 128, device="cuda")
    o = _delta_gpu(k, q, kk, v, a, b, ldab, a_log, dt_bias, states, total, nk, nv, seq_start=_u32(starts), n_seq=len(lens))
    for s, n in enumerate(lens):
        lo, hi = int(starts[s]), int(starts[s + 1])
        st = np.zeros((nv, 128, 128), np.float32)
        want = cpu_ref.gated_delta(np32(q)[lo:hi], np32(kk)[lo:hi], np32(v)[lo:hi], np32(a)[lo:hi], np32(b)[lo:hi], ldab,
                                   np32(a_log), np32(dt_bias), st, n, nk, nv, 128, 128)
        assert_close(np32(o)[lo:hi], want, what=f"packed delta seq {s}", **DELTA_TOL)
        assert_close(np32(states[s]), st, what=f"packed delta state {s}", **DELTA_TOL)


@pytest.mark.parametrize("lens,nk,nv,with_prev", [([1], 16, 16, False), ([70], 16, 16, True), ([130, 5, 64, 200], 16, 16, True), ([90, 33], 8, 16, False)])
def test_conv_gated_delta_fused_equals_the_two_calls(k, lens, nk, nv, with_prev):
    """conv + SiLU + L2 norm inside the delta rule's first kernel (dc_conv_gated_delta) against the oracle's conv followed by
    its sequential delta rule, per sequence, with carried conv rows and two value heads per key head among the cases."""
    if not k.delta.conv_gated_delta_supported():
        pytest.skip("the fused form needs the tcgen05 engine with split 3")
    conv_dim = (2 * nk + nv) * 128
    ldp = conv_dim + nv * 128 + 2 * nv           # qkv | z | b | a, as the fused projection lays them out
    starts = np.concatenate([[0], np.cumsum(lens)])
    total, n_seq = int(starts[-1]), len(lens)
    p = randn(200, total, ldp)
    w = randn(201, conv_dim, 4, std=0.3)
    prev = randn(202, n_seq, 3, conv_dim) if with_prev else None
    a_log = torch.rand(nv, generator=torch.Generator().manual_seed(203)) * 2.7
    dt_bias = 1.0 + randn(204, nv, std=0.02)
    states = torch.zeros(n_seq, nv, 128, 128, device="cuda")
    o = torch.empty(total, nv, 128, device="cuda")
    pd = p.cuda()
    b_col, a_col = conv_dim + nv * 128, conv_dim + nv * 128 + nv
    k.delta.conv_gated_delta(None, pd, prev.cuda() if with_prev else None, w.cuda(), (pd, a_col * 4), (pd, b_col * 4), a_log.cuda(), dt_bias.cuda(),
                             None, states, o, total, ldp, True, nk, nv, seq_start=_u32(starts), n_seq=n_seq, max_len=max(lens))
    k.dev.check_status()
    pn = np32(p)
    for s, n in enumerate(lens):
        lo, hi = int(starts[s]), int(starts[s + 1])
        pv = np32(prev[s]) if with_prev else np.zeros((3, conv_dim), np.float32)
        wq, wk, wv = cpu_ref.conv_silu_l2(pn[lo:hi], ldp, n, pv, np32(w), nk, nv, 128, 128)
        st = np.zeros((nv, 128, 128), np.float32)
        want = cpu_ref.gated_delta(wq, wk, wv, np.ascontiguousarray(pn[lo:hi, a_col:a_col + nv]), np.ascontiguousarray(pn[lo:hi, b_col:b_col + nv]), nv,
                                   np32(a_log), np32(dt_bias), st, n, nk, nv, 128, 128)
        assert_close(np32(o)[lo:hi], want, what=f"fused conv+delta o, seq {s}", **DELTA_TOL)
        assert_close(np32(states[s]), st, what=f"fused conv+delta state, seq {s}", **DELTA_TOL)


@pytest.mark.parametrize("n_seq", [10, 40])
def test_gated_delta_many_sequences_use_wider_lanes(k, n_seq, delta_impl):
    """With many sequences the sequential kernel gives each value column fewer lanes (4, then 1) than for a
    single sequence (8), and the chunked kernel keeps all 128 value columns in one CTA instead of 32;
    every variant must match the sequential reference."""
    nk = nv = 16
    rs = np.random.RandomState(n_seq)
    lens = rs.randint(1, 24, n_seq).tolist()
    if n_seq == 10:
        lens += [30] * 150  # 160 sequences x 16 heads: above the SM count, the one-CTA-per-head variant
    starts = np.concatenate([[0], np.cumsum(lens)])
    total = int(starts[-1])
    q, kk, v, a, b, ldab, a_log, dt_bias = _delta_inputs(120 + n_seq, total, nk, nv)
    n_seq = len(lens)
    states = torch.zeros(n_seq, nv, 128, 128, device="cuda")
    o = _delta_gpu(k, q, kk, v, a, b, ldab, a_log, dt_bias, states, total, nk, nv, seq_start=_u32(starts), n_seq=n_seq, max_len=max(lens))
    for s in (0, n_seq // 2, n_seq - 1):
        lo, hi = int(starts[s]), int(starts[s + 1])
        st = np.zeros((nv, 128, 128), np.float32)
        want = cpu_ref.gated_delta(np32(q)[lo:hi], np32(kk)[lo:hi], np32(v)[lo:hi], np32(a)[lo:hi], np32(b)[lo:hi], ldab,
                                   np32(a_log), np32(dt_bias), st, hi - lo, nk, nv, 128, 128)
        assert_close(np32(o)[lo:hi], want, what=f"delta seq {s} of {n_seq}", **DELTA_TOL)
        assert_close(np32(states[s]), st, what=f"delta state {s} of {n_seq}", **DELTA_TOL)


def test_gated_delta_single_pass_precision(k):
    """The chunked kernel with unsplit bf16 operands (dc_set_delta_split 1) is a looser, faster mode:
    it must still track the reference to bf16 accuracy, and the default split-3 mode must be much closer."""
    t, nk, nv = 200, 16, 16
    q, kk, v, a, b, ldab, a_log, dt_bias = _delta_inputs(300, t, nk, nv)
    st = np.zeros((nv, 128, 128), np.float32)
    want = cpu_ref.gated_delta(np32(q), np32(kk), np32(v), np32(a), np32(b), ldab, np32(a_log), np32(dt_bias), st, t, nk, nv, 128, 128)
    errs = {}
    for split in (3, 1):
        k.dev.set_delta_split(split)
        try:
            o = _delta_gpu(k, q, kk, v, a, b, ldab, a_log, dt_bias, torch.zeros(nv, 128, 128, device="cuda"), t, nk, nv)
        finally:
            k.dev.set_delta_split(3)
        errs[split] = float(np.linalg.norm(np32(o) - want) / np.linalg.norm(want))
    assert errs[3] < 5e-5 and errs[1] < 2e-2 and errs[3] < errs[1] / 20, errs
