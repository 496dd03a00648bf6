"""Per-kernel micro-benchmarks: one operator at one shape, timed with CUDA events.

    python -m decide_b200.bench_ops gemm --m 38592 --n 19456 --k 2560 --epi swiglu
    python -m decide_b200.bench_ops rmsnorm --rows 38592
    python -m decide_b200.bench_ops delta --seqs 64 --tokens 603
    python -m decide_b200.bench_ops request --tokens 603   # ONE request through the whole 36-layer engine
    python -m decide_b200.bench_ops all            # every hot-path kernel at the benchmark's shapes

Prints one JSON line per case: microseconds per launch, the algorithmic work (FLOPs for GEMM and
attention, bytes for the HBM-bound kernels) and the rate that implies. This is the analogue of the
reference's per-kernel profiler and `gemm_lab` sweeps (crates/decide-metal/src/profile.rs:29-101,
gemm_configs.rs:35-36); it is also the small, self-terminating command that `ncu` captures run on.
Inputs are larger than L2 at the default shapes; between launches nothing is flushed on purpose, the
default shapes stream far more than the 126 MB of L2.
"""
from __future__ import annotations

import argparse
import json
import math

import numpy as np
import torch

from .kernels import Device, Epilogue, Kernels

EPI = {"f32": Epilogue.StoreF32, "store16": Epilogue.StoreBF16, "add": Epilogue.AddF32, "swiglu": Epilogue.SwigluBF16}


# (N, K, epilogue) of gate_up, down, the Gated-DeltaNet in- and out-projection, the attention in-projection and o-proj
PROJECTIONS = [(19456, 2560, "swiglu"), (2560, 9728, "add"), (8224, 2560, "f32"), (2560, 2048, "add"), (10240, 2560, "f32"), (2560, 4096, "add")]


def _time(fn, iters: int, warmup: int) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / iters  # microseconds


def _u32(a):
    return torch.as_tensor(np.asarray(a, dtype=np.int32)).cuda()


def _seqs(n_seq, tokens):
    starts = np.arange(n_seq + 1) * tokens
    pos = np.tile(np.arange(tokens), n_seq)
    return _u32(starts), _u32(pos)


def gemm(k: Kernels, m, n, kk, epi: str, iters, warmup, bn=0):
    act = k.dev.act_torch
    x = torch.randn(m, kk, device="cuda").to(act)
    w = (torch.randn(n, kk, device="cuda") * 0.02).to(act)
    e = EPI[epi]
    n_out = n // 2 if e == Epilogue.SwigluBF16 else n
    y = torch.zeros(m, n_out, dtype=torch.float32 if e in (Epilogue.StoreF32, Epilogue.AddF32) else act, device="cuda")
    if bn:
        fn = lambda: k.gemm.gemm_tile(None, x, w, y, m, n, kk, kk, kk, n_out, e, bn)
    else:
        fn = lambda: k.gemm.gemm(None, x, w, y, m, n, kk, kk, kk, n_out, e)
    us = _time(fn, iters, warmup)
    flops = 2.0 * m * n * kk
    plan_bn, tail_split = k.gemm.plan_k(m, n, kk)
    return {"op": "gemm", "m": m, "n": n, "k": kk, "epilogue": epi, "tile_n": bn or plan_bn, "tail_k_split": 1 if bn else tail_split, "us": us, "flops": flops,
            "tflops": flops / us / 1e6}


def rmsnorm(k, rows, h, iters, warmup):
    x = torch.randn(rows, h, device="cuda")
    w = torch.randn(h, device="cuda") * 0.02
    y = torch.empty(rows, h, dtype=k.dev.act_torch, device="cuda")
    us = _time(lambda: k.norm.rmsnorm(None, x, w, y, None, rows, h, h, h, True), iters, warmup)
    nbytes = rows * h * 6.0
    return {"op": "rmsnorm", "rows": rows, "h": h, "us": us, "bytes": nbytes, "gbs": nbytes / us / 1e3}


def gnorm(k, rows, nv, iters, warmup):
    ldz = 6144 + nv * 128 + 2 * nv
    o = torch.randn(rows, nv * 128, device="cuda")
    p = torch.randn(rows, ldz, device="cuda")
    w = torch.ones(128, device="cuda")
    y = torch.empty(rows, nv * 128, dtype=k.dev.act_torch, device="cuda")
    us = _time(lambda: k.gnorm.gated_rmsnorm_silu(None, o, (p, 6144 * 4), w, y, rows, ldz, nv), iters, warmup)
    nbytes = rows * nv * 128 * 10.0
    return {"op": "gated_rmsnorm_silu", "rows": rows, "us": us, "bytes": nbytes, "gbs": nbytes / us / 1e3}


def conv(k, n_seq, tokens, nk, nv, iters, warmup):
    rows = n_seq * tokens
    conv_dim = (2 * nk + nv) * 128
    ldp = conv_dim + nv * 128 + 2 * nv
    p = torch.randn(rows, ldp, device="cuda")
    w = torch.randn(conv_dim, 4, device="cuda") * 0.3
    q = torch.empty(rows, nk, 128, device="cuda")
    kk = torch.empty(rows, nk, 128, device="cuda")
    v = torch.empty(rows, nv, 128, device="cuda")
    starts, _ = _seqs(n_seq, tokens)
    us = _time(lambda: k.conv.conv_silu_l2(None, p, None, w, q, kk, v, rows, ldp, nk, nv, seq_start=starts, n_seq=n_seq, max_len=tokens), iters, warmup)
    nbytes = rows * conv_dim * 8.0
    return {"op": "conv_silu_l2", "rows": rows, "us": us, "bytes": nbytes, "gbs": nbytes / us / 1e3}


def delta(k, n_seq, tokens, nk, nv, iters, warmup, impl="fast", split=3, engine="tcgen05"):
    from .kernels import Engine, Family, Impl
    k.dev.set_impl(Family.Delta, Impl.Fast if impl == "fast" else Impl.Baseline)
    k.dev.set_delta_split(split)
    k.dev.set_engine(Family.Delta, Engine.Tcgen05 if engine == "tcgen05" else Engine.MmaSync)
    rows = n_seq * tokens
    q = torch.nn.functional.normalize(torch.randn(rows, nk, 128, device="cuda"), dim=-1) * 128 ** -0.5
    kk = torch.nn.functional.normalize(torch.randn(rows, nk, 128, device="cuda"), dim=-1)
    v = torch.randn(rows, nv, 128, device="cuda")
    ab = torch.randn(rows, 2 * nv, device="cuda")
    a_log = torch.rand(nv, device="cuda") * math.log(16.0)
    dt = torch.ones(nv, device="cuda")
    o = torch.empty(rows, nv, 128, device="cuda")
    starts, _ = _seqs(n_seq, tokens)
    fn = lambda: k.delta.gated_delta(None, q, kk, v, (ab, nv * 4), ab, a_log, dt, None, None, o, rows, 2 * nv, False, nk, nv, seq_start=starts, n_seq=n_seq, max_len=tokens)
    us = _time(fn, iters, warmup)
    k.dev.set_impl(Family.Delta, Impl.Fast)
    k.dev.set_delta_split(3)
    k.dev.set_engine(Family.Delta, Engine.Tcgen05)
    nbytes = rows * (2 * nk + 2 * nv) * 128 * 4.0
    flops = rows * nv * 128.0 * 128.0 * 7.0  # the sequential recurrence: decay, two dots, rank-1 update per state element
    return {"op": "gated_delta", "impl": impl if impl != "fast" else f"chunked split {split}" + (f" {engine}" if split == 3 else ""), "seqs": n_seq, "tokens": tokens, "us": us, "bytes": nbytes, "gbs": nbytes / us / 1e3, "flops": flops, "tflops_fp32": flops / us / 1e6,
            "us_per_token_step": us / tokens}


def conv_delta(k, n_seq, tokens, nk, nv, iters, warmup, fused=True):
    """conv + SiLU + L2 norm and the gated delta rule over a random fused projection buffer [rows, qkv|z|b|a]:
    in one call (dc_conv_gated_delta) or as the two calls."""
    rows = n_seq * tokens
    conv_dim = (2 * nk + nv) * 128
    ldp = conv_dim + nv * 128 + 2 * nv
    p = torch.randn(rows, ldp, device="cuda")
    w = torch.randn(conv_dim, 4, device="cuda") * 0.3
    a_log = torch.rand(nv, device="cuda") * math.log(16.0)
    dt = torch.ones(nv, device="cuda")
    o = torch.empty(rows, nv, 128, device="cuda")
    starts, _ = _seqs(n_seq, tokens)
    b_col, a_col = conv_dim + nv * 128, conv_dim + nv * 128 + nv
    if fused:
        fn = lambda: k.delta.conv_gated_delta(None, p, None, w, (p, a_col * 4), (p, b_col * 4), a_log, dt, None, None, o, rows, ldp, False, nk, nv,
                                              seq_start=starts, n_seq=n_seq, max_len=tokens)
    else:
        q = torch.empty(rows, nk, 128, device="cuda")
        kk = torch.empty_like(q)
        v = torch.empty(rows, nv, 128, device="cuda")

        def fn():
            k.conv.conv_silu_l2(None, p, None, w, q, kk, v, rows, ldp, nk, nv, seq_start=starts, n_seq=n_seq, max_len=tokens)
            k.delta.gated_delta(None, q, kk, v, (p, a_col * 4), (p, b_col * 4), a_log, dt, None, None, o, rows, ldp, False, nk, nv,
                                seq_start=starts, n_seq=n_seq, max_len=tokens)
    us = _time(fn, iters, warmup)
    return {"op": "conv+gated_delta", "impl": "one call" if fused else "two calls", "seqs": n_seq, "tokens": tokens, "us": us}


def rope(k, rows, nq, nkv, gated, iters, warmup):
    hd = 128
    ld = (2 if gated else 1) * nq * hd + 2 * nkv * hd
    p = torch.randn(rows, ld, device="cuda")
    w = torch.randn(hd, device="cuda") * 0.02
    inv = torch.tensor([1e6 ** (-2.0 * i / hd) for i in range(hd // 2)], device="cuda")
    pos = _u32(np.arange(rows) % 603)
    act = k.dev.act_torch
    qo = torch.empty(rows, nq, hd, dtype=act, device="cuda")
    kc = torch.empty(rows, nkv, hd, dtype=act, device="cuda")
    vc = torch.empty(rows, nkv, hd, dtype=act, device="cuda")
    kcol = (2 if gated else 1) * nq * hd

    def fn():
        k.rope.q_norm_rope(None, p, w, inv, pos, qo, rows, ld, nq, hd, hd)
        k.rope.kv_norm_rope(None, p, w, inv, kc, vc, rows, ld, kcol, kcol + nkv * hd, 0, rows, nkv, hd, hd, pos=pos)

    us = _time(fn, iters, warmup)
    nbytes = rows * (nq + 2 * nkv) * hd * 6.0
    return {"op": "q_norm_rope+kv_norm_rope", "rows": rows, "us": us, "bytes": nbytes, "gbs": nbytes / us / 1e3}


def attention(k, n_seq, tokens, nq, nkv, gated, iters, warmup):
    hd, rows = 128, n_seq * tokens
    act = k.dev.act_torch
    q = torch.randn(rows, nq, hd, device="cuda").to(act)
    kc = torch.randn(rows, nkv, hd, device="cuda").to(act)
    vc = torch.randn(rows, nkv, hd, device="cuda").to(act)
    gate = torch.randn(rows, nq * hd, device="cuda") if gated else None
    y = torch.empty(rows, nq * hd, dtype=act, device="cuda")
    starts, pos = _seqs(n_seq, tokens)
    fn = lambda: k.attn.attention(None, q, kc, vc, gate, pos, y, rows, nq * hd, nq, nkv, hd, seq_start=starts, n_seq=n_seq, max_len=tokens)
    us = _time(fn, iters, warmup)
    flops = 4.0 * hd * nq * n_seq * tokens * (tokens + 1) / 2
    return {"op": "attention", "seqs": n_seq, "tokens": tokens, "gated": gated, "us": us, "flops": flops, "tflops": flops / us / 1e6}


def config_case(k: Kernels, cfg: int, iters: int, warmup: int, gated: bool = True) -> dict:
    """One of the benchmark's single-block configs as an op SEQUENCE on the GPU (weights ~N(0, 0.02), inputs ~N(0, 1)):
      0  gate_up GEMM with SwiGLU, M = 276             1  MLP block, M = 603: RMSNorm -> gate_up (SwiGLU) -> down (+ residual)
      2  attention layer, M = 2,307: RMSNorm -> in-projection -> q/k norm + RoPE -> causal GQA attention -> o-projection + residual
      3  Gated DeltaNet layer, M = 2,307: RMSNorm -> in-projection -> conv + SiLU + L2 + chunk-64 delta rule -> gated RMSNorm -> out-projection + residual
    Returns microseconds per pass and the algorithmic FLOPs of its GEMMs (+ the attention core)."""
    act = k.dev.act_torch
    H, I, nq, nkv, hd, nk, nv = 2560, 9728, 32, 8, 128, 16, 16
    g = torch.Generator(device="cuda").manual_seed(cfg)
    rn = lambda *shape, std=1.0: torch.randn(*shape, generator=g, device="cuda") * std
    wmat = lambda n, kk: rn(n, kk, std=0.02).to(act)
    m = {0: 276, 1: 603, 2: 2307, 3: 2307}[cfg]
    x = rn(m, H)
    h = torch.empty(m, H, dtype=act, device="cuda")
    nw = rn(H, std=0.02)
    norm = lambda: k.norm.rmsnorm(None, x, nw, h, None, m, H, H, H, True)
    if cfg in (0, 1):
        w_gu, w_down = wmat(2 * I, H), wmat(H, I)
        mlp = torch.empty(m, I, dtype=act, device="cuda")
        gu = lambda: k.gemm.gemm(None, h, w_gu, mlp, m, 2 * I, H, H, H, I, Epilogue.SwigluBF16)
        if cfg == 0:
            h.copy_(rn(m, H).to(act))
            fn, flops, what = gu, 2.0 * m * 2 * I * H, "gate_up GEMM + SwiGLU"
        else:
            def fn():
                norm()
                gu()
                k.gemm.gemm(None, mlp, w_down, x, m, H, I, I, I, H, Epilogue.AddF32)
            flops, what = 2.0 * m * 2 * I * H + 2.0 * m * H * I, "RMSNorm -> gate_up (SwiGLU) -> down + residual"
    elif cfg == 2:
        qd, kvd = nq * hd, nkv * hd
        n_in = (2 if gated else 1) * qd + 2 * kvd
        w_in, w_o = wmat(n_in, H), wmat(H, qd)
        p = torch.empty(m, n_in, device="cuda")
        qw, kw = rn(hd, std=0.02), rn(hd, std=0.02)
        inv = torch.tensor([1e6 ** (-2.0 * i / hd) for i in range(hd // 2)], device="cuda")
        starts, pos = _seqs(1, m)
        qo = torch.empty(m, nq, hd, dtype=act, device="cuda")
        kc, vc = torch.empty(m, nkv, hd, dtype=act, device="cuda"), torch.empty(m, nkv, hd, dtype=act, device="cuda")
        y = torch.empty(m, qd, dtype=act, device="cuda")
        kcol = (2 if gated else 1) * qd

        def fn():
            norm()
            k.gemm.gemm(None, h, w_in, p, m, n_in, H, H, H, n_in, Epilogue.StoreF32)
            k.rope.q_norm_rope(None, p, qw, inv, pos, qo, m, n_in, nq, hd, hd)
            k.rope.kv_norm_rope(None, p, kw, inv, kc, vc, m, n_in, kcol, kcol + kvd, 0, m, nkv, hd, hd, pos=pos)
            k.attn.attention(None, qo, kc, vc, (p, qd * 4) if gated else None, pos, y, m, n_in, nq, nkv, hd, seq_start=starts, n_seq=1, max_len=m)
            k.gemm.gemm(None, y, w_o, x, m, H, qd, qd, qd, H, Epilogue.AddF32)
        flops = 2.0 * m * n_in * H + 2.0 * m * H * qd + 4.0 * hd * nq * m * (m + 1) / 2
        what = f"attention layer, {'gated (N = 10240)' if gated else 'un-gated (N = 6144)'}"
    else:
        conv_dim, vd = (2 * nk + nv) * 128, nv * 128
        n_in = conv_dim + vd + 2 * nv
        w_in, w_out = wmat(n_in, H), wmat(H, vd)
        p = torch.empty(m, n_in, device="cuda")
        cw = rn(conv_dim, 4, std=0.3)
        a_log = torch.rand(nv, generator=g, device="cuda") * math.log(16.0)
        dt, gw = torch.ones(nv, device="cuda"), torch.ones(128, device="cuda")
        o = torch.empty(m, nv, 128, device="cuda")
        gg = torch.empty(m, vd, dtype=act, device="cuda")
        starts, _ = _seqs(1, m)
        b_col, a_col = conv_dim + vd, conv_dim + vd + nv

        def fn():
            norm()
            k.gemm.gemm(None, h, w_in, p, m, n_in, H, H, H, n_in, Epilogue.StoreF32)
            k.delta.conv_gated_delta(None, p, None, cw, (p, a_col * 4), (p, b_col * 4), a_log, dt, None, None, o, m, n_in, False, nk, nv,
                                     seq_start=starts, n_seq=1, max_len=m)
            k.gnorm.gated_rmsnorm_silu(None, o, (p, conv_dim * 4), gw, gg, m, n_in, nv)
            k.gemm.gemm(None, gg, w_out, x, m, H, vd, vd, vd, H, Epilogue.AddF32)
        flops, what = 2.0 * m * n_in * H + 2.0 * m * H * vd, "Gated DeltaNet layer"
    us = _time(fn, iters, warmup)
    k.dev.check_status()
    return {"config": cfg, "what": what, "rows": m, "us": us, "flops": flops, "tflops": flops / us / 1e6}


def request(dev: Device, tokens: int, iters: int, warmup: int) -> dict:
    """One request of `tokens` token ids through the full synthetic 36-layer model, host ids in, host logits out (the
    single-request latency of the benchmark; DECIDE_GRAPHS=0 enqueues kernel by kernel, which a launch list wants)."""
    from .engine import Engine
    from .synth import synth_batch, synth_fused_on_device
    from .weights import BASELINE_DIMS as dims

    cuda = torch.device("cuda", 0)
    fused, embed, final_norm = synth_fused_on_device(dims, 1, cuda)
    eng = Engine(dims, dev=dev, max_rows=max(4096, tokens), max_seqs=1, max_answers=8, max_cand=16, fused_layers=fused, embed=embed, final_norm=final_norm)
    one = synth_batch(dims, 1, tokens, seed=7, n_answers=6 if tokens < 1000 else 3, n_cand=16, max_cand=16)
    l0 = dev.launches
    eng.logits(one)
    per_forward = dev.launches - l0
    us = _time(lambda: eng.logits(one), iters, warmup)
    out = {"op": "request", "tokens": tokens, "rows_run": eng.resident_rows, "us": us, "launches_per_forward": per_forward, "graphs": eng.graph_count}
    eng.close()
    return out


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("op", choices=["gemm", "gemms", "rowwise", "rmsnorm", "gnorm", "conv", "delta", "conv_delta", "rope", "attention", "request", "all"])
    ap.add_argument("--m", type=int, default=38592)
    ap.add_argument("--n", type=int, default=19456)
    ap.add_argument("--k", type=int, default=2560)
    ap.add_argument("--epi", choices=list(EPI), default="swiglu")
    ap.add_argument("--bn", type=int, default=0, help="force the GEMM tile width (128 or 256)")
    ap.add_argument("--rows", type=int, default=38592)
    ap.add_argument("--seqs", type=int, default=64)
    ap.add_argument("--tokens", type=int, default=603)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    a = ap.parse_args()
    dev = Device(0)
    k = Kernels(dev)
    out = []
    if a.op == "gemm":
        out.append(gemm(k, a.m, a.n, a.k, a.epi, a.iters, a.warmup, a.bn))
    elif a.op == "gemms":   # the six projection shapes of the model at --m rows
        for (n, kk, epi) in PROJECTIONS:
            out.append(gemm(k, a.m, n, kk, epi, a.iters, a.warmup))
    elif a.op == "rowwise":  # the memory-bound kernels at --rows rows
        out += [rmsnorm(k, a.rows, 2560, a.iters, a.warmup), gnorm(k, a.rows, 16, a.iters, a.warmup), rope(k, a.rows, 32, 8, True, a.iters, a.warmup)]
    elif a.op == "rmsnorm":
        out.append(rmsnorm(k, a.rows, 2560, a.iters, a.warmup))
    elif a.op == "gnorm":
        out.append(gnorm(k, a.rows, 16, a.iters, a.warmup))
    elif a.op == "conv":
        out.append(conv(k, a.seqs, a.tokens, 16, 16, a.iters, a.warmup))
    elif a.op == "delta":
        out.append(delta(k, a.seqs, a.tokens, 16, 16, a.iters, a.warmup))
        out.append(delta(k, a.seqs, a.tokens, 16, 16, a.iters, a.warmup, engine="mma"))
    elif a.op == "conv_delta":
        out.append(conv_delta(k, a.seqs, a.tokens, 16, 16, a.iters, a.warmup))
        out.append(conv_delta(k, a.seqs, a.tokens, 16, 16, a.iters, a.warmup, fused=False))
    elif a.op == "rope":
        out.append(rope(k, a.rows, 32, 8, True, a.iters, a.warmup))
    elif a.op == "attention":
        out.append(attention(k, a.seqs, a.tokens, 32, 8, True, a.iters, a.warmup))
    elif a.op == "request":
        out.append(request(dev, a.tokens, a.iters, a.warmup))
    else:
        for m in (603, 2307, 38592):
            for (n, kk, epi) in PROJECTIONS:
                out.append(gemm(k, m, n, kk, epi, a.iters, a.warmup))
        for seqs, tokens in ((64, 603), (1, 2307)):
            rows = seqs * tokens
            out += [rmsnorm(k, rows, 2560, a.iters, a.warmup), gnorm(k, rows, 16, a.iters, a.warmup), conv(k, seqs, tokens, 16, 16, a.iters, a.warmup),
                    delta(k, seqs, tokens, 16, 16, a.iters, a.warmup), delta(k, seqs, tokens, 16, 16, a.iters, a.warmup, engine="mma"),
                    delta(k, seqs, tokens, 16, 16, a.iters, a.warmup, split=1),
                    delta(k, seqs, tokens, 16, 16, a.iters, a.warmup, impl="baseline"), conv_delta(k, seqs, tokens, 16, 16, a.iters, a.warmup),
                    conv_delta(k, seqs, tokens, 16, 16, a.iters, a.warmup, fused=False), rope(k, rows, 32, 8, True, a.iters, a.warmup),
                    attention(k, seqs, tokens, 32, 8, True, a.iters, a.warmup)]
    dev.check_status()
    for r in out:
        print(json.dumps(r))


if __name__ == "__main__":
    main()
