"""The engine's op sequence over the restated cpu_ref functions, on the CPU.

TEST INFRASTRUCTURE ONLY (see oracle/cpu_ref.py). It composes oracle/cpu_ref.py in the order of
the reference's Forward (crates/decide-engine/src/forward.rs:1191-1276 encode_layer / encode_mlp,
1312-1328 head) over weights in the engine's fused layouts, with fp32 activations everywhere
(`round_bf16=True` or `round_to="bf16" | "f16"` additionally rounds the GEMM inputs and 16-bit
intermediates the way the engine stores them; `exact_inputs` names GEMMs whose input is NOT
rounded, which is what feeding that GEMM the activation as a hi + lo pair of 16-bit values does). Its purpose is to tie the two oracles together: tests check that this composition
agrees with the Hugging Face model code that reference/gold.py runs, which pins both the restated
kernels' semantics and the fused weight layouts without a GPU. Slow; small cases only.
"""
from __future__ import annotations

import numpy as np

from . import cpu_ref

f32 = np.float32


def _w(t):
    return t.detach().float().cpu().numpy()


def f16_round(a):
    """Round-to-nearest-even f32 -> fp16 -> f32."""
    return np.asarray(a, dtype=f32).astype(np.float16).astype(f32)


def forward_logits(d, fused_layers, embed, final_norm, ids, positions, cands, round_bf16: bool = False, layer_outputs=None,
                   round_to: str | None = None, exact_inputs: tuple = (), all_reduce=None):
    """One request: ids [T] -> list of logits arrays (one per answer position).

    exact_inputs: subset of ("in", "out", "gate_up", "down"): the projections whose 16-bit input is kept exact.
    all_reduce: for one rank's shard of a tensor-parallel group (d and fused_layers are the shard's): a function that
    sums an fp32 array over the ranks; it is applied to the out and down projections before they join the residual."""
    ar = all_reduce or (lambda a: a)
    if round_bf16:
        round_to = "bf16"
    rnd = {None: (lambda a: a), "bf16": cpu_ref.bf16_round, "f16": f16_round}[round_to]
    r = rnd

    def rin(name, a):
        return a if name in exact_inputs else rnd(a)
    t = len(ids)
    emb = _w(embed)
    x = emb[np.asarray(ids, dtype=np.int64)].astype(f32)
    pos = np.arange(t)
    for l, lw in enumerate(fused_layers):
        h = rin("in", cpu_ref.rmsnorm(x, _w(lw["in_norm"]), d.hidden, True))
        if not d.is_full_attention(l):
            ld = d.lin_in_n
            p = cpu_ref.gemm_nt(h, _w(lw["w_in"]), t, ld, d.hidden)
            q, k, v = cpu_ref.conv_silu_l2(p, ld, t, np.zeros((3, d.conv_dim), f32), _w(lw["conv_w"]), d.gdn_nk, d.gdn_nv, d.gdn_dk, d.gdn_dv)
            b = p[:, d.conv_dim + d.value_dim:d.conv_dim + d.value_dim + d.gdn_nv]
            a = p[:, d.conv_dim + d.value_dim + d.gate_cols:d.conv_dim + d.value_dim + d.gate_cols + d.gdn_nv]
            state = np.zeros((d.gdn_nv, d.gdn_dv, d.gdn_dk), f32)
            o = cpu_ref.gated_delta(q, k, v, a, b, d.gdn_nv, _w(lw["a_log"]), _w(lw["dt_bias"]), state, t, d.gdn_nk, d.gdn_nv, d.gdn_dk, d.gdn_dv)
            z = np.ascontiguousarray(p[:, d.conv_dim:d.conv_dim + d.value_dim])
            g = rin("out", cpu_ref.gated_rmsnorm_silu(o, z, d.value_dim, _w(lw["gnorm"]), t, d.gdn_nv, d.gdn_dv))
            out_k = d.value_dim
        else:
            ld = d.att_in_n
            p = cpu_ref.gemm_nt(h, _w(lw["w_in"]), t, ld, d.hidden)
            kcol = 2 * d.q_dim if d.attn_gate else d.q_dim
            vcol = kcol + d.kv_dim
            qh = p[:, :d.q_dim].reshape(t, d.nq, d.head_dim)
            kh = p[:, kcol:kcol + d.kv_dim].reshape(t, d.nkv, d.head_dim)
            qo = r(cpu_ref.head_norm_rope(qh, _w(lw["q_norm"]), pos[:, None].repeat(d.nq, 1), d.rot_dim, d.rope_theta))
            kc = r(cpu_ref.head_norm_rope(kh, _w(lw["k_norm"]), pos[:, None].repeat(d.nkv, 1), d.rot_dim, d.rope_theta))
            vc = r(p[:, vcol:vcol + d.kv_dim].reshape(t, d.nkv, d.head_dim))
            gate = p[:, d.q_dim:2 * d.q_dim] if d.attn_gate else None
            g = rin("out", cpu_ref.attention(qo, pos, kc, vc, gate, d.nq, d.nkv, d.head_dim))
            out_k = d.q_dim
        x = (x + ar(cpu_ref.gemm_nt(g, _w(lw["w_out"]), t, d.hidden, out_k))).astype(f32)
        h = rin("gate_up", cpu_ref.rmsnorm(x, _w(lw["post_norm"]), d.hidden, True))
        gu = cpu_ref.gemm_nt(h, _w(lw["w_gu"]), t, 2 * d.inter, d.hidden)
        mlp = rin("down", cpu_ref.swiglu_interleaved(gu, t, 2 * d.inter, d.swiglu_block))
        x = (x + ar(cpu_ref.gemm_nt(mlp, _w(lw["w_down"]), t, d.hidden, d.inter))).astype(f32)
        if layer_outputs is not None:
            layer_outputs.append(x.copy())
    xs = x[np.asarray(positions, dtype=np.int64)]
    cand_rows = [emb[np.asarray(c, dtype=np.int64)] for c in cands]
    return cpu_ref.final_head(xs, _w(final_norm), cand_rows, d.hidden)
