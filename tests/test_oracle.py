"""CPU tests of the oracle itself (oracle/cpu_ref.py): the reference's three by-hand known-answer
tests (crates/decide-engine/src/cpu_ref.rs:204-236) restated, plus internal consistency checks that
need no GPU (chunk continuation of the conv and the delta rule, RoPE against a direct formula)."""
import math

import numpy as np

from oracle import cpu_ref

f32 = np.float32


def test_rmsnorm_by_hand():
    # cpu_ref.rs:204-211: mean(x^2) = 12.5, (1 + w) = 2
    y = cpu_ref.rmsnorm(np.array([3.0, 4.0], f32), np.array([1.0, 1.0], f32), 2, True)
    assert abs(y[0, 0] - 3.0 * 2.0 / math.sqrt(12.5)) < 1e-5
    assert abs(y[0, 1] - 4.0 * 2.0 / math.sqrt(12.5)) < 1e-5


def test_swiglu_pairs_blocks():
    # cpu_ref.rs:213-220
    blk = 16
    y = np.zeros(2 * blk, f32)
    y[3] = 1.0
    y[blk + 3] = 2.0
    out = cpu_ref.swiglu_interleaved(y, 1, 2 * blk, blk)[0]
    assert abs(out[3] - float(cpu_ref.silu(1.0)) * 2.0) < 1e-6
    assert all(v == 0.0 for i, v in enumerate(out) if i != 3)


def test_delta_rule_with_unit_gate_is_a_delta_update():
    # cpu_ref.rs:222-236, reference dims NK=16, NV=32
    nk, nv, dk, dv = 16, 32, 128, 128
    state = np.zeros((nv, dv, dk), f32)
    k = np.zeros((1, nk, dk), f32)
    k[0, 0, 0] = 1.0
    v = np.zeros((1, nv, dv), f32)
    v[0, 0, 5] = 3.0
    a, b = np.zeros((1, nv), f32), np.full((1, nv), 50.0, f32)
    o = cpu_ref.gated_delta(k.copy(), k, v, a, b, nv, np.full(nv, -np.inf, f32), np.zeros(nv, f32), state, 1, nk, nv, dk, dv)
    assert abs(o[0, 0, 5] - 3.0) < 1e-5
    assert abs(state[0, 5, 0] - 3.0) < 1e-5


def test_gemm_nt_matches_float64_matmul():
    rs = np.random.RandomState(0)
    x, w = rs.randn(5, 32).astype(f32), rs.randn(7, 32).astype(f32)
    assert np.array_equal(cpu_ref.gemm_nt(x, w, 5, 7, 32), (x.astype(np.float64) @ w.astype(np.float64).T).astype(f32))


def test_conv_chunks_carry_state():
    rs = np.random.RandomState(1)
    nk = nv = 2
    conv_dim = (2 * nk + nv) * 128
    t, ldp = 11, conv_dim + 8
    p = rs.randn(t, ldp).astype(f32)
    w = rs.randn(conv_dim, 4).astype(f32)
    zero = np.zeros((3, conv_dim), f32)
    q, k, v = cpu_ref.conv_silu_l2(p, ldp, t, zero, w, nk, nv, 128, 128)
    cut = 4
    q1, k1, v1 = cpu_ref.conv_silu_l2(p[:cut], ldp, cut, zero, w, nk, nv, 128, 128)
    prev = cpu_ref.conv_state_update(p[:cut], ldp, cut, zero, conv_dim)
    q2, k2, v2 = cpu_ref.conv_silu_l2(p[cut:], ldp, t - cut, prev, w, nk, nv, 128, 128)
    assert np.array_equal(np.concatenate([q1, q2]), q)
    assert np.array_equal(np.concatenate([v1, v2]), v)
    # q is unit-norm times dk^-1/2, k unit-norm
    assert np.allclose(np.linalg.norm(q, axis=-1), 128 ** -0.5, atol=1e-4)
    assert np.allclose(np.linalg.norm(k, axis=-1), 1.0, atol=1e-4)


def test_delta_chunks_carry_state():
    rs = np.random.RandomState(2)
    t, nk, nv = 9, 2, 4
    q, k = rs.randn(t, nk, 128).astype(f32), rs.randn(t, nk, 128).astype(f32)
    k /= np.linalg.norm(k, axis=-1, keepdims=True)
    v = rs.randn(t, nv, 128).astype(f32)
    a, b = rs.randn(t, nv).astype(f32), rs.randn(t, nv).astype(f32)
    a_log, dtb = rs.rand(nv).astype(f32), np.ones(nv, f32)
    s = np.zeros((nv, 128, 128), f32)
    o = cpu_ref.gated_delta(q, k, v, a, b, nv, a_log, dtb, s, t, nk, nv, 128, 128)
    s2 = np.zeros((nv, 128, 128), f32)
    o1 = cpu_ref.gated_delta(q[:4], k[:4], v[:4], a[:4], b[:4], nv, a_log, dtb, s2, 4, nk, nv, 128, 128)
    o2 = cpu_ref.gated_delta(q[4:], k[4:], v[4:], a[4:], b[4:], nv, a_log, dtb, s2, t - 4, nk, nv, 128, 128)
    assert np.array_equal(np.concatenate([o1, o2]), o) and np.array_equal(s, s2)


def test_rope_is_a_rotation_and_identity_at_position_zero():
    rs = np.random.RandomState(3)
    seg = rs.randn(6, 128).astype(f32)
    w = np.zeros(128, f32)
    at0 = cpu_ref.head_norm_rope(seg, w, np.zeros(6), 128, 1e6)
    normed = cpu_ref.rmsnorm(seg, w, 128, True)
    assert np.allclose(at0, normed, atol=1e-6)
    at9 = cpu_ref.head_norm_rope(seg, w, np.full(6, 9), 128, 1e6)
    assert np.allclose(np.linalg.norm(at9, axis=-1), np.linalg.norm(normed, axis=-1), rtol=1e-5)
    # partial rotary leaves the tail alone
    part = cpu_ref.head_norm_rope(seg, w, np.full(6, 9), 32, 1e6)
    assert np.array_equal(part[:, 32:], normed[:, 32:])


def test_attention_single_position_returns_v():
    rs = np.random.RandomState(4)
    q = rs.randn(1, 4, 128).astype(f32)
    kc, vc = rs.randn(1, 2, 128).astype(f32), rs.randn(1, 2, 128).astype(f32)
    out = cpu_ref.attention(q, [0], kc, vc, None, 4, 2, 128).reshape(4, 128)
    assert np.allclose(out[0], vc[0, 0]) and np.allclose(out[3], vc[0, 1])


def test_bf16_round_matches_torch():
    import torch

    x = np.random.RandomState(5).randn(1000).astype(f32)
    assert np.array_equal(cpu_ref.bf16_round(x), torch.from_numpy(x).to(torch.bfloat16).float().numpy())
