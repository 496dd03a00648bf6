"""Seeded synthetic weights and requests.

The real checkpoint, tokenizer and request fixtures of the reference cannot be used here, so the
model is random-initialised at the given dims and requests are random token ids; everything is a
pure function of a seed, generated on the CPU in fp32 and rounded to bf16 where the tensor is bf16,
so that the CPU reference forward and the GPU engine see the same bits.

Distributions: Linear and embedding weights ~N(0, 0.02) (the architecture's default init), norm
weights zero-centred ~N(0, 0.02) (effective 1 + w), the gated-norm weight 1 + N(0, 0.02), conv taps
~N(0, 0.02), A_log ~U(0, ln 16), dt_bias 1 + N(0, 0.02), token ids ~U[0, vocab).
Tensor names are the checkpoint's (Hugging Face Qwen3.5 text model), which is what the converter of
the reference reads (crates/decide-engine/src/convert.rs:204-245).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np
import torch

from .weights import Dims


def _gen(seed: int) -> torch.Generator:
    return torch.Generator().manual_seed(seed)


def _normal(g, *shape, std=0.02, mean=0.0, dtype=torch.float32):
    t = torch.empty(*shape, dtype=torch.float32).normal_(mean, std, generator=g)
    return t.to(dtype)


def synth_layer(d: Dims, layer: int, seed: int) -> dict:
    """One layer's checkpoint-layout tensors. A layer's values depend only on (seed, layer)."""
    g = _gen(seed * 100003 + layer + 1)
    p = f"layers.{layer}."
    bf = torch.bfloat16
    sd = {
        p + "input_layernorm.weight": _normal(g, d.hidden),
        p + "post_attention_layernorm.weight": _normal(g, d.hidden),
        p + "mlp.gate_proj.weight": _normal(g, d.inter, d.hidden, dtype=bf),
        p + "mlp.up_proj.weight": _normal(g, d.inter, d.hidden, dtype=bf),
        p + "mlp.down_proj.weight": _normal(g, d.hidden, d.inter, dtype=bf),
    }
    if d.is_full_attention(layer):
        a = p + "self_attn."
        sd[a + "q_proj.weight"] = _normal(g, (2 if d.attn_gate else 1) * d.q_dim, d.hidden, dtype=bf)
        sd[a + "k_proj.weight"] = _normal(g, d.kv_dim, d.hidden, dtype=bf)
        sd[a + "v_proj.weight"] = _normal(g, d.kv_dim, d.hidden, dtype=bf)
        sd[a + "o_proj.weight"] = _normal(g, d.hidden, d.q_dim, dtype=bf)
        sd[a + "q_norm.weight"] = _normal(g, d.head_dim)
        sd[a + "k_norm.weight"] = _normal(g, d.head_dim)
    else:
        a = p + "linear_attn."
        sd[a + "in_proj_qkv.weight"] = _normal(g, d.conv_dim, d.hidden, dtype=bf)
        sd[a + "in_proj_z.weight"] = _normal(g, d.value_dim, d.hidden, dtype=bf)
        sd[a + "in_proj_b.weight"] = _normal(g, d.gdn_nv, d.hidden, dtype=bf)
        sd[a + "in_proj_a.weight"] = _normal(g, d.gdn_nv, d.hidden, dtype=bf)
        sd[a + "conv1d.weight"] = _normal(g, d.conv_dim, 1, 4)
        sd[a + "A_log"] = torch.empty(d.gdn_nv).uniform_(0.0, math.log(16.0), generator=g)
        sd[a + "dt_bias"] = _normal(g, d.gdn_nv, mean=1.0)
        sd[a + "norm.weight"] = _normal(g, d.gdn_dv, mean=1.0)
        sd[a + "out_proj.weight"] = _normal(g, d.hidden, d.value_dim, dtype=bf)
    return sd


def synth_globals(d: Dims, seed: int) -> dict:
    g = _gen(seed * 100003)
    return {"embed_tokens.weight": _normal(g, d.vocab, d.hidden, dtype=torch.bfloat16), "norm.weight": _normal(g, d.hidden)}


def synth_state_dict(d: Dims, seed: int) -> dict:
    sd = synth_globals(d, seed)
    for l in range(d.n_layers):
        sd.update(synth_layer(d, l, seed))
    return sd


@dataclass
class Batch:
    """A batch of requests in the engine's input form: packed ids, per-request offsets, answer rows
    (packed row indices), candidate ids per answer row."""
    ids: np.ndarray          # uint32 [rows]
    seq_start: np.ndarray    # uint32 [n_seq + 1]
    ans_rows: np.ndarray     # uint32 [n_ans]
    cand: np.ndarray         # uint32 [n_ans, max_cand]
    ncand: np.ndarray        # uint32 [n_ans]

    @property
    def n_seq(self): return len(self.seq_start) - 1
    @property
    def rows(self): return int(self.seq_start[-1])


# Answer rows of a request of T tokens: the spacing of the reference's 603-token `ticket6` fixture
# (tests/fixtures/gold/fp32/core/ticket6.json: positions 551..596 of 603), counted from the end.
ANSWER_OFFSETS_FROM_END = (52, 44, 33, 25, 16, 7)


def synth_batch(d: Dims, n_req: int, tokens: int, seed: int, n_answers: int = 6, n_cand: int = 16, max_cand: int = 16) -> Batch:
    rs = np.random.RandomState(seed)
    ids = rs.randint(0, d.vocab, size=n_req * tokens).astype(np.uint32)
    seq_start = (np.arange(n_req + 1) * tokens).astype(np.uint32)
    offs = [o for o in ANSWER_OFFSETS_FROM_END if o <= tokens][-n_answers:]
    if len(offs) < n_answers:  # short requests: the last rows
        offs = list(range(min(n_answers, tokens), 0, -1))
    ans = np.array([r * tokens + tokens - o for r in range(n_req) for o in offs], dtype=np.uint32)
    cand = np.zeros((len(ans), max_cand), dtype=np.uint32)
    for i in range(len(ans)):
        cand[i, :n_cand] = rs.choice(d.vocab, size=n_cand, replace=False)
    ncand = np.full(len(ans), n_cand, dtype=np.uint32)
    return Batch(ids, seq_start, ans, cand, ncand)


def synth_fused_on_device(d: Dims, seed: int, device) -> tuple[list, torch.Tensor, torch.Tensor]:
    """Random-init weights drawn directly on the GPU in the engine's fused layouts (same distributions
    as `synth_layer`, different bits): for throughput runs, where no CPU copy is needed.
    Returns (fused layers, embedding table, final norm weight)."""
    g = torch.Generator(device=device).manual_seed(seed)
    bf = torch.bfloat16

    def normal(*shape, std=0.02, mean=0.0, dtype=torch.float32):
        return torch.empty(*shape, dtype=torch.float32, device=device).normal_(mean, std, generator=g).to(dtype)

    layers = []
    for l in range(d.n_layers):
        lw = {"in_norm": normal(d.hidden), "post_norm": normal(d.hidden), "w_gu": normal(2 * d.inter, d.hidden, dtype=bf),
              "w_down": normal(d.hidden, d.inter, dtype=bf)}
        if d.is_full_attention(l):
            lw.update(w_in=normal(d.att_in_n, d.hidden, dtype=bf), w_out=normal(d.hidden, d.q_dim, dtype=bf),
                      q_norm=normal(d.head_dim), k_norm=normal(d.head_dim))
        else:
            lw.update(w_in=normal(d.lin_in_n, d.hidden, dtype=bf), w_out=normal(d.hidden, d.value_dim, dtype=bf),
                      conv_w=normal(d.conv_dim, 4),
                      a_log=torch.empty(d.gdn_nv, device=device).uniform_(0.0, math.log(16.0), generator=g),
                      dt_bias=normal(d.gdn_nv, mean=1.0), gnorm=normal(d.gdn_dv, mean=1.0))
        layers.append(lw)
    return layers, normal(d.vocab, d.hidden, dtype=bf), normal(d.hidden)
