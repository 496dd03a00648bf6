"""The fp32 CPU gold forward of the reference, on synthetic weights.

TEST INFRASTRUCTURE ONLY (see oracle/cpu_ref.py): the checker and the timed CPU baseline, never
part of the product path.

The reference's parity target is `reference/gold.py --mode fp32`: the model code of the Hugging Face
`transformers` Qwen3.5 text model on the CPU with every op in fp32 (gold.py:32-63): Linear weights
stay bf16 and are upcast per call (gold.py:57-60), every other parameter is fp32, the embedding
output is upcast (gold.py:61-62); then `hidden[positions] @ emb[cands].float().T` (gold.py:126-133).
gold.py itself cannot run here: it imports InternLM's `inference.py` and loads the
Intern-Decision-4B checkpoint, neither of which ships with the reference. What can run is the same
model class from the installed `transformers` (the arithmetic lives in that third-party package:
`transformers.models.qwen3_5.modeling_qwen3_5`, reference pin 5.14.1, installed 5.5.0), built from
a synthetic config and fed seeded random weights. This module does exactly that and nothing else;
the model source is imported, not copied.

Parity pin: UNPINNED by the reference's own golden vectors for the logits (those need the real
checkpoint). Pinned indirectly: this module and oracle/cpu_ref.py (the restated cpu_ref.rs) are
independent statements of the same layer math and tests/ check that they agree.
"""
from __future__ import annotations

import time
import types

import numpy as np
import torch
import torch.nn as nn
import torch.nn.functional as F


def hf_config(d):
    from transformers.models.qwen3_5.configuration_qwen3_5 import Qwen3_5TextConfig

    if not d.attn_gate:
        raise ValueError("the Qwen3.5 attention class always has the output gate")
    return Qwen3_5TextConfig(
        vocab_size=d.vocab, hidden_size=d.hidden, intermediate_size=d.inter, num_hidden_layers=d.n_layers,
        num_attention_heads=d.nq, num_key_value_heads=d.nkv, head_dim=d.head_dim, linear_conv_kernel_dim=4,
        linear_key_head_dim=d.gdn_dk, linear_value_head_dim=d.gdn_dv, linear_num_key_heads=d.gdn_nk,
        linear_num_value_heads=d.gdn_nv, rms_norm_eps=d.eps, tie_word_embeddings=True, hidden_act="silu",
        full_attention_interval=d.full_attn_interval, attn_output_gate=True, attention_bias=False,
        rope_parameters={"rope_type": "default", "rope_theta": d.rope_theta, "partial_rotary_factor": d.rot_dim / d.head_dim},
        max_position_embeddings=32768, attn_implementation="sdpa")


def build_model(d, state_dict: dict):
    """Qwen3_5TextModel with `state_dict` (checkpoint names; bf16 Linear/Embedding weights, fp32 the
    rest), computing as gold.py's fp32 mode does."""
    from transformers.models.qwen3_5 import modeling_qwen3_5 as mq

    # torch-only code paths (gold.py runs on a CPU where the fused kernels are absent)
    for name in ("FusedRMSNormGated", "chunk_gated_delta_rule", "fused_recurrent_gated_delta_rule", "causal_conv1d_fn", "causal_conv1d_update"):
        if getattr(mq, name, None) is not None:
            setattr(mq, name, None)
    cfg = hf_config(d)
    assert [("full_attention" if d.is_full_attention(i) else "linear_attention") for i in range(d.n_layers)] == list(cfg.layer_types)
    with torch.device("meta"):
        model = mq.Qwen3_5TextModel(cfg)
    missing, unexpected = model.load_state_dict(state_dict, strict=False, assign=True)
    assert not unexpected, unexpected
    assert all("rotary_emb" in k for k in missing), missing
    model.rotary_emb = mq.Qwen3_5TextRotaryEmbedding(cfg)  # its buffers are not in the checkpoint
    model.eval()

    def linear_fp32(self, x):  # gold.py:57-60
        return F.linear(x.float(), self.weight.float(), None if self.bias is None else self.bias.float())

    for mod in model.modules():
        if isinstance(mod, nn.Linear):
            mod.forward = types.MethodType(linear_fp32, mod)
        elif not isinstance(mod, nn.Embedding):
            for name, p in list(mod.named_parameters(recurse=False)):
                assert p.dtype == torch.float32, (name, p.dtype)  # gold.py:45-55: non-Linear params are fp32
    embed_forward = model.embed_tokens.forward
    model.embed_tokens.forward = lambda ids: embed_forward(ids).float()  # gold.py:61-62
    return model


@torch.inference_mode()
def gold_hidden(model, ids: np.ndarray, hooks=None) -> torch.Tensor:
    """Final-norm hidden states [T, hidden] of one request (gold.py:128)."""
    t = torch.from_numpy(np.asarray(ids, dtype=np.int64))[None]
    hidden = model(input_ids=t, use_cache=False).last_hidden_state[0]
    assert hidden.dtype == torch.float32
    return hidden


@torch.inference_mode()
def gold_logits(model, ids: np.ndarray, positions, cands) -> tuple[list, float]:
    """Candidate logits of one request and the seconds it took, as gold.py:126-133 times them:
    forward + `hidden[pos] @ emb[cands].float().T`."""
    t0 = time.perf_counter()
    hidden = gold_hidden(model, ids)
    emb = model.get_input_embeddings().weight
    out = [(hidden[int(p)] @ emb[torch.as_tensor(np.asarray(c, dtype=np.int64))].float().T).numpy() for p, c in zip(positions, cands)]
    return out, time.perf_counter() - t0


@torch.inference_mode()
def gold_layer_outputs(model, ids: np.ndarray) -> list:
    """The residual stream after every layer (gold.py:115-118 hooks), as float32 arrays [T, hidden]."""
    captured = []
    hooks = [layer.register_forward_hook(lambda m, a, out: captured.append((out[0] if isinstance(out, tuple) else out).detach()[0].numpy().copy()))
             for layer in model.layers]
    try:
        gold_hidden(model, ids)
    finally:
        for h in hooks:
            h.remove()
    return captured


def gold_batch_logits(model, batch, max_cand: int) -> tuple[np.ndarray, float]:
    """Logits [n_ans, max_cand] (unused entries 0) for a packed batch, request by request; returns the
    total forward seconds as well."""
    out = np.zeros((len(batch.ans_rows), max_cand), dtype=np.float32)
    total = 0.0
    for s in range(batch.n_seq):
        lo, hi = int(batch.seq_start[s]), int(batch.seq_start[s + 1])
        idx = [i for i, r in enumerate(batch.ans_rows) if lo <= r < hi]
        positions = [int(batch.ans_rows[i]) - lo for i in idx]
        cands = [batch.cand[i, :batch.ncand[i]] for i in idx]
        logits, sec = gold_logits(model, batch.ids[lo:hi], positions, cands)
        total += sec
        for i, l in zip(idx, logits):
            out[i, :len(l)] = l
    return out, total
