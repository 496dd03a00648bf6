"""CPU restatement of decide's per-kernel reference, `crates/decide-engine/src/cpu_ref.rs`.

TEST INFRASTRUCTURE ONLY. This module is the checker for the CUDA kernels: only `tests/`,
`__graft_entry__.smoke()` and the CPU-baseline leg of `bench.py` may import it. Nothing in
`decide_b200/` does, and the product has no CPU path.

Each function follows the Rust function of the same name (file:line given per function):
f32 storage, f64 accumulation inside dot products and mean-squares, `(ms as f32) + eps` before the
square root, the L2 norm's eps inside the sqrt, DK^-1/2 on q only, RoPE pairs (i, i + rot/2).
The reference compiles its model dims in (config.rs:4-37); here they are arguments, because the
benchmark configs use other dims than the reference's checkpoint. numpy vectorises the loops the
Rust spells out; the arithmetic per element is the same.

Pinned by: the reference's three by-hand known-answer tests (cpu_ref.rs:204-236), restated in
tests/test_oracle.py, and by agreement with the HF model code the reference's gold generator runs
(reference/gold.py:126-133) on seeded inputs, also in tests/.
"""
from __future__ import annotations

import numpy as np

EPS = np.float32(1e-6)  # config.rs:33

f32 = np.float32
f64 = np.float64


def silu(x):  # cpu_ref.rs:6
    x = np.asarray(x, dtype=f32)
    return (x / (f32(1.0) + np.exp(-x, dtype=f32))).astype(f32)


def sigmoid(x):  # cpu_ref.rs:7
    x = np.asarray(x, dtype=f32)
    return (f32(1.0) / (f32(1.0) + np.exp(-x, dtype=f32))).astype(f32)


def softplus(x):  # cpu_ref.rs:8
    x = np.asarray(x, dtype=f32)
    with np.errstate(over="ignore"):
        return np.where(x > f32(20.0), x, np.log(f32(1.0) + np.exp(x, dtype=f32), dtype=f32)).astype(f32)


def rmsnorm(x, w, h: int, add_one: bool, eps=EPS):
    """cpu_ref.rs:11-22. x [rows*h] or [rows,h] f32 -> [rows,h] f32."""
    x = np.asarray(x, dtype=f32).reshape(-1, h)
    w = np.asarray(w, dtype=f32)
    ms = (x.astype(f64) ** 2).sum(axis=1) / h
    inv = (f32(1.0) / np.sqrt(ms.astype(f32) + f32(eps), dtype=f32)).astype(f32)
    wv = (f32(1.0) + w) if add_one else w
    return (x * inv[:, None] * wv[None, :]).astype(f32)


def gemm_nt(x, w, m: int, n: int, k: int):
    """cpu_ref.rs:25-36. y[m][n] = sum_k x[m][k] w[n][k], f64 accumulation, f32 result."""
    x = np.asarray(x, dtype=f32).reshape(m, k).astype(f64)
    w = np.asarray(w, dtype=f32).reshape(n, k).astype(f64)
    return (x @ w.T).astype(f32)


def swiglu_interleaved(y, m: int, n2: int, block: int = 16):
    """cpu_ref.rs:39-50. [m, n2] interleaved gate|up blocks -> [m, n2/2]."""
    y = np.asarray(y, dtype=f32).reshape(m, n2 // (2 * block), 2, block)
    g, u = y[:, :, 0, :], y[:, :, 1, :]
    return (silu(g) * u).astype(f32).reshape(m, n2 // 2)


def conv_silu_l2(p, ldp: int, t: int, prev, w, nk: int, nv: int, dk: int, dv: int, conv_k: int = 4):
    """cpu_ref.rs:55-81. Returns (q [t,nk,dk], k [t,nk,dk], v [t,nv,dv])."""
    key_dim, value_dim = nk * dk, nv * dv
    conv_dim = 2 * key_dim + value_dim
    p = np.asarray(p, dtype=f32).reshape(t, ldp)[:, :conv_dim]
    prev = np.asarray(prev, dtype=f32).reshape(conv_k - 1, conv_dim)
    w = np.asarray(w, dtype=f32).reshape(conv_dim, conv_k)
    raw = np.concatenate([prev, p], axis=0).astype(f64)  # row s of the chunk is raw[s + 3]
    acc = np.zeros((t, conv_dim), dtype=f64)
    for j in range(conv_k):
        acc += w[:, j].astype(f64)[None, :] * raw[j:j + t]
    y = silu(acc.astype(f32))

    def l2(seg, scale):
        ss = (seg.astype(f64) ** 2).sum(axis=-1)
        inv = (f32(1.0) / np.sqrt(ss.astype(f32) + f32(1e-6), dtype=f32)).astype(f32)
        return (seg * inv[..., None] * f32(scale)).astype(f32)

    q = l2(y[:, :key_dim].reshape(t, nk, dk), f32(dk) ** f32(-0.5))
    k = l2(y[:, key_dim:2 * key_dim].reshape(t, nk, dk), f32(1.0))
    v = y[:, 2 * key_dim:].reshape(t, nv, dv).copy()
    return q, k, v


def conv_state_update(p, ldp: int, t: int, prev, conv_dim: int):
    """cpu_ref.rs:86-95. The 3 raw rows that end the chunk, oldest first."""
    p = np.asarray(p, dtype=f32).reshape(t, ldp)[:, :conv_dim]
    prev = np.asarray(prev, dtype=f32).reshape(3, conv_dim)
    return np.concatenate([prev, p], axis=0)[-3:].copy()


def gated_delta(q, k, v, a, b, ldab: int, a_log, dt_bias, state, t: int, nk: int, nv: int, dk: int, dv: int):
    """cpu_ref.rs:101-129: the sequential gated delta rule. `state` [nv,dv,dk] f32 is updated in place.

    a, b are [t, ldab] (value head h at column h). Returns o [t,nv,dv].
    """
    q = np.asarray(q, dtype=f32).reshape(t, nk, dk)
    k = np.asarray(k, dtype=f32).reshape(t, nk, dk)
    v = np.asarray(v, dtype=f32).reshape(t, nv, dv)
    a = np.asarray(a, dtype=f32).reshape(t, ldab)
    b = np.asarray(b, dtype=f32).reshape(t, ldab)
    a_log = np.asarray(a_log, dtype=f32)
    dt_bias = np.asarray(dt_bias, dtype=f32)
    assert state.shape == (nv, dv, dk) and state.dtype == f32
    rep = nv // nk
    hk = np.arange(nv) // rep
    o = np.zeros((t, nv, dv), dtype=f32)
    for s in range(t):
        with np.errstate(over="ignore"):
            g = np.exp(-(np.exp(a_log, dtype=f32)) * softplus(a[s, :nv] + dt_bias), dtype=f32)  # [nv]
        beta = sigmoid(b[s, :nv])
        kt = k[s, hk]  # [nv, dk]
        qt = q[s, hk]
        state *= g[:, None, None]
        kv = np.einsum("hvk,hk->hv", state.astype(f64), kt.astype(f64))
        delta = ((v[s] - kv.astype(f32)) * beta[:, None]).astype(f32)  # [nv, dv]
        state += (kt[:, None, :] * delta[:, :, None]).astype(f32)
        o[s] = np.einsum("hvk,hk->hv", state.astype(f64), qt.astype(f64)).astype(f32)
    return o


def gated_rmsnorm_silu(o, z, ldz: int, w, t: int, nv: int, dv: int, eps=EPS):
    """cpu_ref.rs:132-145. o [t,nv,dv], z rows of stride ldz -> y [t, nv*dv]."""
    o = np.asarray(o, dtype=f32).reshape(t, nv, dv)
    z = np.asarray(z, dtype=f32).reshape(t, ldz)[:, :nv * dv].reshape(t, nv, dv)
    w = np.asarray(w, dtype=f32)
    ms = (o.astype(f64) ** 2).sum(axis=-1) / dv
    inv = (f32(1.0) / np.sqrt(ms.astype(f32) + f32(eps), dtype=f32)).astype(f32)
    return (o * inv[..., None] * w[None, None, :] * silu(z)).astype(f32).reshape(t, nv * dv)


def inv_freq(rot_dim: int, theta: float):
    """config.rs:44-46: 1 / theta^(2i/rot) in f32."""
    i = np.arange(rot_dim // 2, dtype=f32)
    return (f32(1.0) / np.power(f32(theta), (f32(2.0) * i) / f32(rot_dim), dtype=f32)).astype(f32)


def head_norm_rope(seg, w, pos, rot_dim: int, theta: float, eps=EPS):
    """cpu_ref.rs:149-162, for many segments at once. seg [..., hd], pos broadcastable to seg[..., 0]."""
    seg = np.asarray(seg, dtype=f32)
    hd = seg.shape[-1]
    w = np.asarray(w, dtype=f32)
    ms = (seg.astype(f64) ** 2).sum(axis=-1) / hd
    inv = (f32(1.0) / np.sqrt(ms.astype(f32) + f32(eps), dtype=f32)).astype(f32)
    x = (seg * inv[..., None] * (f32(1.0) + w)).astype(f32)
    f = inv_freq(rot_dim, theta)
    ang = (np.asarray(pos, dtype=f32)[..., None] * f).astype(f32)  # fp32 angle
    sn = np.sin(ang.astype(f64)).astype(f32)
    cs = np.cos(ang.astype(f64)).astype(f32)
    half = rot_dim // 2
    a_, b_ = x[..., :half].copy(), x[..., half:rot_dim].copy()
    x[..., :half] = a_ * cs - b_ * sn
    x[..., half:rot_dim] = b_ * cs + a_ * sn
    return x


def attention(q, qpos, kc, vc, gate, nq: int, nkv: int, hd: int):
    """cpu_ref.rs:167-188. q [rows,nq,hd]; kc, vc [npos,nkv,hd]; gate [rows,nq*hd] or None.

    Row r attends to cache rows 0..=qpos[r]; scale hd^-1/2; f64 softmax.
    """
    q = np.asarray(q, dtype=f32).reshape(-1, nq, hd)
    kc = np.asarray(kc, dtype=f32).reshape(-1, nkv, hd)
    vc = np.asarray(vc, dtype=f32).reshape(-1, nkv, hd)
    rows = q.shape[0]
    out = np.zeros((rows, nq * hd), dtype=f32)
    rep = nq // nkv
    scale = f64(hd) ** -0.5
    for s in range(rows):
        n = int(qpos[s]) + 1
        for h in range(nq):
            kvh = h // rep
            sc = (kc[:n, kvh].astype(f64) @ q[s, h].astype(f64)) * scale
            e = np.exp(sc - sc.max())
            acc = e @ vc[:n, kvh].astype(f64)
            out[s, h * hd:(h + 1) * hd] = (acc / e.sum()).astype(f32)
    if gate is not None:
        out = (out * sigmoid(np.asarray(gate, dtype=f32).reshape(rows, nq * hd))).astype(f32)
    return out


def final_head(x, w, candidates, h: int):
    """cpu_ref.rs:192-198. x [rows,h]; candidates[r] = [ncand_r, h] f32 (bf16 rows widened)."""
    normed = rmsnorm(x, w, h, True)
    return [(np.asarray(c, dtype=f32).astype(f64) @ normed[r].astype(f64)).astype(f32) for r, c in enumerate(candidates)]


def bf16_round(x):
    """Round-to-nearest-even f32 -> bf16 -> f32, so the reference sees what the GPU sees
    (the idiom of the reference's test helpers, crates/decide-engine/src/testutil.rs:10-12)."""
    u = np.asarray(x, dtype=f32).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    return r.astype(np.uint32).view(f32)
