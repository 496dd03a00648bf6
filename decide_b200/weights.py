"""Model dims and the fused weight layouts the kernels read.

The reference compiles its dims in (crates/decide-engine/src/config.rs:4-41) and fuses the
checkpoint's tensors at conversion time (crates/decide-engine/src/convert.rs:35-62, 204-245):
  linear layer   w_in = in_proj_qkv | in_proj_z | in_proj_b | in_proj_a      (rows)
  attention      w_in = q rows | gate rows | k_proj | v_proj, the checkpoint's q_proj being
                 per head [head_dim query rows, head_dim gate rows]
  MLP            w_gu = gate_proj and up_proj rows interleaved in blocks of 16
Here the dims are a value (`Dims`) and the same fusions are applied to a state dict with the
checkpoint's (Hugging Face Qwen3.5 text model) tensor names. Matrices are bf16 (the reference
converts to fp16), small tensors fp32.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class Dims:
    hidden: int = 2560
    n_layers: int = 36
    nq: int = 32
    nkv: int = 8
    head_dim: int = 128
    rot_dim: int = 128
    gdn_nk: int = 16
    gdn_nv: int = 16
    gdn_dk: int = 128
    gdn_dv: int = 128
    inter: int = 9728
    vocab: int = 151936
    full_attn_interval: int = 4
    attn_gate: bool = True
    swiglu_block: int = 16
    eps: float = 1e-6
    rope_theta: float = 1e6

    # derived sizes, named as in config.rs
    @property
    def key_dim(self): return self.gdn_nk * self.gdn_dk
    @property
    def value_dim(self): return self.gdn_nv * self.gdn_dv
    @property
    def conv_dim(self): return 2 * self.key_dim + self.value_dim
    @property
    def gate_cols(self): return -(-self.gdn_nv // 16) * 16   # columns of each of the b and a blocks: gdn_nv rounded up to 16
    @property
    def lin_in_n(self): return self.conv_dim + self.value_dim + 2 * self.gate_cols
    @property
    def q_dim(self): return self.nq * self.head_dim
    @property
    def kv_dim(self): return self.nkv * self.head_dim
    @property
    def att_in_n(self): return (2 if self.attn_gate else 1) * self.q_dim + 2 * self.kv_dim

    def is_full_attention(self, layer: int) -> bool:  # config.rs:39-41
        return (layer + 1) % self.full_attn_interval == 0

    def tp_local(self, world: int) -> "Dims":
        """The dims of one rank's shard in a tensor-parallel group of `world`: heads and the intermediate size divided,
        hidden size, layer count and vocabulary whole."""
        for name in ("nq", "nkv", "gdn_nk", "gdn_nv"):
            if getattr(self, name) % world:
                raise ValueError(f"{name} = {getattr(self, name)} does not divide over {world} ranks")
        if self.inter % (32 * world):
            raise ValueError(f"inter = {self.inter} must split into multiples of 32 over {world} ranks")
        return Dims(**{**self.__dict__, "nq": self.nq // world, "nkv": self.nkv // world, "gdn_nk": self.gdn_nk // world,
                       "gdn_nv": self.gdn_nv // world, "inter": self.inter // world})

    def gemm_flops_per_row(self) -> float:
        """2*N*K summed over the projection GEMMs of all layers, per token row."""
        total = 0.0
        for l in range(self.n_layers):
            if self.is_full_attention(l):
                total += 2.0 * self.hidden * self.att_in_n + 2.0 * self.q_dim * self.hidden
            else:
                total += 2.0 * self.hidden * self.lin_in_n + 2.0 * self.value_dim * self.hidden
            total += 2.0 * self.hidden * 2 * self.inter + 2.0 * self.inter * self.hidden
        return total


    def gemm_flops(self, rows: int, n_ans: int, pruned: bool) -> float:
        """2*M*N*K over the projection GEMMs of one forward of `rows` rows; with `pruned`, the last (attention) layer
        runs its k|v projection over all rows and everything else over the n_ans answer rows only."""
        if not (pruned and self.is_full_attention(self.n_layers - 1)):
            return self.gemm_flops_per_row() * rows
        last = 2.0 * self.hidden * self.att_in_n + 2.0 * self.q_dim * self.hidden + 2.0 * self.hidden * 2 * self.inter + 2.0 * self.inter * self.hidden
        kv = 2.0 * self.hidden * 2 * self.kv_dim
        return (self.gemm_flops_per_row() - last) * rows + kv * rows + (last - kv) * n_ans


# The dims the benchmark configs use, and the reference checkpoint's own dims cut to what the kernels
# support (head_dim 128 only), for a second tested instantiation.
BASELINE_DIMS = Dims()


class CDims(ctypes.Structure):
    """dc_dims of include/decide_cuda.h."""
    _fields_ = [(n, ctypes.c_uint32) for n in (
        "hidden", "n_layers", "nq", "nkv", "head_dim", "rot_dim", "gdn_nk", "gdn_nv", "gdn_dk", "gdn_dv", "inter", "vocab",
        "full_attn_interval", "attn_gate", "swiglu_block")] + [("eps", ctypes.c_float), ("rope_theta", ctypes.c_float)]

    @classmethod
    def of(cls, d: Dims) -> "CDims":
        return cls(d.hidden, d.n_layers, d.nq, d.nkv, d.head_dim, d.rot_dim, d.gdn_nk, d.gdn_nv, d.gdn_dk, d.gdn_dv, d.inter,
                   d.vocab, d.full_attn_interval, int(d.attn_gate), d.swiglu_block, d.eps, d.rope_theta)


LAYER_FIELDS = ("in_norm", "w_in", "w_out", "post_norm", "w_gu", "w_down", "conv_w", "a_log", "dt_bias", "gnorm", "q_norm", "k_norm")


class CLayerWeights(ctypes.Structure):
    """dc_layer_weights of include/decide_cuda.h."""
    _fields_ = [(n, ctypes.c_void_p) for n in LAYER_FIELDS]


def deinterleave_q_gate(q_proj: torch.Tensor, heads: int, head_dim: int) -> torch.Tensor:
    """Per-head [query rows, gate rows] -> [all query rows | all gate rows] (convert.rs:35-47)."""
    k = q_proj.shape[1]
    v = q_proj.reshape(heads, 2, head_dim, k)
    return torch.cat([v[:, 0].reshape(heads * head_dim, k), v[:, 1].reshape(heads * head_dim, k)], dim=0)


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor, block: int) -> torch.Tensor:
    """gate_proj and up_proj rows interleaved in blocks of `block` rows (convert.rs:49-62)."""
    n, k = gate.shape
    assert up.shape == gate.shape and n % block == 0, f"gate/up must be equal [n, k] matrices with n a multiple of {block}"
    return torch.stack([gate.reshape(n // block, block, k), up.reshape(n // block, block, k)], dim=1).reshape(2 * n, k)


def fuse_layer(sd: dict, i: int, d: Dims) -> dict:
    """One layer's tensors in the engine's layouts, from checkpoint names (convert.rs:204-245)."""
    bf = lambda t: t.to(torch.bfloat16).contiguous()
    f32 = lambda t: t.to(torch.float32).contiguous()
    p = f"layers.{i}."
    out = {"in_norm": f32(sd[p + "input_layernorm.weight"]), "post_norm": f32(sd[p + "post_attention_layernorm.weight"])}
    if d.is_full_attention(i):
        q = sd[p + "self_attn.q_proj.weight"]
        if d.attn_gate:
            assert q.shape == (2 * d.q_dim, d.hidden)
            q = deinterleave_q_gate(q, d.nq, d.head_dim)
        out["w_in"] = bf(torch.cat([q, sd[p + "self_attn.k_proj.weight"], sd[p + "self_attn.v_proj.weight"]], dim=0))
        out["q_norm"] = f32(sd[p + "self_attn.q_norm.weight"])
        out["k_norm"] = f32(sd[p + "self_attn.k_norm.weight"])
        out["w_out"] = bf(sd[p + "self_attn.o_proj.weight"])
        assert out["w_in"].shape == (d.att_in_n, d.hidden)
    else:
        la = p + "linear_attn."
        pad = torch.zeros(d.gate_cols - d.gdn_nv, d.hidden, dtype=sd[la + "in_proj_b.weight"].dtype)   # b and a blocks are 16 columns wide
        out["w_in"] = bf(torch.cat([sd[la + "in_proj_qkv.weight"], sd[la + "in_proj_z.weight"], sd[la + "in_proj_b.weight"], pad,
                                    sd[la + "in_proj_a.weight"], pad], dim=0))
        out["conv_w"] = f32(sd[la + "conv1d.weight"].reshape(d.conv_dim, 4))
        out["a_log"] = f32(sd[la + "A_log"])
        out["dt_bias"] = f32(sd[la + "dt_bias"])
        out["gnorm"] = f32(sd[la + "norm.weight"])
        out["w_out"] = bf(sd[la + "out_proj.weight"])
        assert out["w_in"].shape == (d.lin_in_n, d.hidden)
    out["w_gu"] = bf(interleave_gate_up(sd[p + "mlp.gate_proj.weight"], sd[p + "mlp.up_proj.weight"], d.swiglu_block))
    out["w_down"] = bf(sd[p + "mlp.down_proj.weight"])
    return out


def tp_shard_layer(lw: dict, layer: int, d: Dims, world: int, rank: int) -> dict:
    """Rank `rank`'s slice of one layer in the fused layouts (`lw` = fuse_layer's output for the whole model, `d` the
    whole model's dims): in-projections and gate_up split by output row (per head, per gate|up block), out and down
    projections by input column, per-head vectors by head; norm weights are replicated. The result is a fused layer of
    the dims `d.tp_local(world)`, so that the sum over ranks of the out / down projections is the unsplit layer's.
    The reference's precedent: the two-way split of each MLP between GPU and Neural Engine
    (crates/decide-engine/src/forward.rs:270-303; convert.rs's ANE split set)."""
    loc = d.tp_local(world)
    rows = lambda t, lo, n: t[lo:lo + n].clone()   # a shard owns its memory: the engine converts matrices in place, and the whole may be freed
    out = {"in_norm": lw["in_norm"], "post_norm": lw["post_norm"]}
    if d.is_full_attention(layer):
        hd = d.head_dim
        parts = [rows(lw["w_in"], rank * loc.q_dim, loc.q_dim)]
        off = d.q_dim
        if d.attn_gate:
            parts.append(rows(lw["w_in"], off + rank * loc.q_dim, loc.q_dim))
            off += d.q_dim
        parts.append(rows(lw["w_in"], off + rank * loc.kv_dim, loc.kv_dim))
        parts.append(rows(lw["w_in"], off + d.kv_dim + rank * loc.kv_dim, loc.kv_dim))
        out["w_in"] = torch.cat(parts, dim=0).contiguous()
        out["w_out"] = lw["w_out"][:, rank * loc.q_dim:(rank + 1) * loc.q_dim].clone()
        out["q_norm"], out["k_norm"] = lw["q_norm"], lw["k_norm"]
        assert out["w_in"].shape[0] == loc.att_in_n and hd == loc.head_dim
    else:
        kd, vd = d.key_dim, d.value_dim
        seg = [(0, rank * loc.key_dim, loc.key_dim), (kd, rank * loc.key_dim, loc.key_dim), (2 * kd, rank * loc.value_dim, loc.value_dim)]
        dev = lw["w_in"].device
        conv_rows = torch.cat([torch.arange(base + lo, base + lo + n, device=dev) for base, lo, n in seg])
        gate_pad = torch.zeros(loc.gate_cols - loc.gdn_nv, lw["w_in"].shape[1], dtype=lw["w_in"].dtype, device=dev)
        b0 = d.conv_dim + vd
        out["w_in"] = torch.cat([lw["w_in"][conv_rows], rows(lw["w_in"], d.conv_dim + rank * loc.value_dim, loc.value_dim),
                                 rows(lw["w_in"], b0 + rank * loc.gdn_nv, loc.gdn_nv), gate_pad,
                                 rows(lw["w_in"], b0 + d.gate_cols + rank * loc.gdn_nv, loc.gdn_nv), gate_pad], dim=0).contiguous()
        out["conv_w"] = lw["conv_w"][conv_rows].contiguous()
        out["a_log"] = rows(lw["a_log"], rank * loc.gdn_nv, loc.gdn_nv)
        out["dt_bias"] = rows(lw["dt_bias"], rank * loc.gdn_nv, loc.gdn_nv)
        out["gnorm"] = lw["gnorm"]
        out["w_out"] = lw["w_out"][:, rank * loc.value_dim:(rank + 1) * loc.value_dim].clone()
        assert out["w_in"].shape[0] == loc.lin_in_n
    out["w_gu"] = rows(lw["w_gu"], rank * 2 * loc.inter, 2 * loc.inter)
    out["w_down"] = lw["w_down"][:, rank * loc.inter:(rank + 1) * loc.inter].clone()
    return out
