"""The operator interface of decide's engine, over the CUDA library.

Mirrors crates/decide-engine/src/kernels/mod.rs:40-67 of the reference: a `Kernels` object holding
one object per kernel family (`k.gemm`, `k.norm`, `k.rope`, ...), one method per kernel, the same
argument order and meaning. Where the reference passes a Metal compute encoder, these take a CUDA
stream (`None` = torch's current stream); where it passes `(buffer, byte offset)` pairs, these take
`(tensor, byte offset)` pairs or plain tensors. Methods only enqueue; nothing synchronises.
Contract violations raise `KernelError` (the reference panics via `assert!`).

torch is used for device memory and streams only; every operation runs in libdecide_cuda.so.
"""
from __future__ import annotations

import ctypes
import enum

import torch

from . import _lib

EPS = 1e-6  # crates/decide-engine/src/config.rs:33


class KernelError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"[dc error {code}] {message}")
        self.code = code


class Epilogue(enum.IntEnum):
    """kernels/gemm.rs:16-26, with bf16 in place of fp16."""
    StoreF32 = 0
    StoreBF16 = 1
    AddF32 = 2
    SwigluBF16 = 3


class Impl(enum.IntEnum):
    """GemmImpl / AttnImpl / DeltaImpl of the reference."""
    Fast = 0
    Baseline = 1


class Family(enum.IntEnum):
    Gemm = 0
    Attn = 1
    Delta = 2


class Act(enum.IntEnum):
    """The context's 16-bit type (DC_ACT_*): activations and weight matrices alike."""
    BF16 = 0
    F16 = 1


class Engine(enum.IntEnum):
    """Tensor-core engine of a family's fast kernels (DC_ENGINE_*)."""
    MmaSync = 0
    Tcgen05 = 1


class ConvertReport(ctypes.Structure):
    """dc_convert_report: the converter's fp16 precision-loss counters (convert.rs:64-71)."""
    _fields_ = [(n, ctypes.c_uint64) for n in ("values", "f16_subnormal", "f16_flushed_to_zero", "f16_overflow")]

    def as_dict(self):
        return {n: int(getattr(self, n)) for n, _ in self._fields_}


def _ptr(arg) -> int:
    """Device address of a tensor, or of (tensor, byte offset); None -> NULL."""
    if arg is None:
        return 0
    if isinstance(arg, tuple):
        t, off = arg
        return t.data_ptr() + int(off)
    return arg.data_ptr()


def _stream(stream) -> int:
    if stream is None:
        return torch.cuda.current_stream().cuda_stream
    return stream.cuda_stream if hasattr(stream, "cuda_stream") else int(stream)


class Device:
    """One context per GPU: the analogue of DecideDevice::shared (crates/decide-metal/src/device.rs:125-130)."""

    def __init__(self, device: int = 0):
        self.lib = _lib.load()
        if not torch.cuda.is_available():
            raise RuntimeError("decide_b200 needs a CUDA device (B200, sm_100a); there is no CPU path")
        torch.cuda.set_device(device)
        torch.cuda.init()
        err = ctypes.create_string_buffer(512)
        self.handle = self.lib.dc_open(device, err, len(err))
        if not self.handle:
            raise RuntimeError(err.value.decode() or "dc_open failed")
        self.device = device

    def close(self):
        if getattr(self, "handle", None):
            self.lib.dc_close(self.handle)
            self.handle = None

    def __del__(self):  # pragma: no cover
        try:
            self.close()
        except Exception:
            pass

    def last_error(self) -> str:
        buf = ctypes.create_string_buffer(1024)
        self.lib.dc_last_error(self.handle, buf, len(buf))
        return buf.value.decode()

    def call(self, name: str, *args):
        rc = getattr(self.lib, name)(self.handle, *args)
        if rc != 0:
            raise KernelError(rc, self.last_error())

    def check_status(self, stream=None):
        """Synchronises the stream and raises if a kernel's bounded wait ran out."""
        self.call("dc_check_status", _stream(stream))

    def selftest_wait_timeout(self, stream=None):
        """Enqueues a kernel whose bounded wait must run out (400 ms); the next check_status raises a DC_TIMEOUT KernelError."""
        self.call("dc_selftest_wait_timeout", _stream(stream))

    def set_impl(self, family: Family, impl: Impl):
        self.call("dc_set_impl", int(family), int(impl))

    def get_impl(self, family: Family) -> Impl:
        return Impl(self.lib.dc_get_impl(self.handle, int(family)))

    def set_activation_dtype(self, act: Act):
        self.call("dc_set_activation_dtype", int(act))

    def set_delta_split(self, split: int):
        """Operand precision of the chunked delta rule: 3 = hi/lo split (default), 1 = single bf16 pass."""
        self.call("dc_set_delta_split", split)

    def set_engine(self, family: Family, engine: "Engine"):
        """Tensor-core engine of the family's fast kernels (attention, delta rule): tcgen05 (default) or mma.sync."""
        self.call("dc_set_engine", int(family), int(engine))

    @property
    def act(self) -> Act:
        return Act(self.lib.dc_get_activation_dtype(self.handle))

    @property
    def act_torch(self) -> torch.dtype:
        """torch dtype of the 16-bit activation buffers this context reads and writes."""
        return torch.float16 if self.act == Act.F16 else torch.bfloat16

    def convert_bf16_to_f16(self, t: torch.Tensor, report: ConvertReport | None = None) -> torch.Tensor:
        """Converts a bf16 device tensor to fp16 IN PLACE and returns it viewed as fp16; adds the
        precision-loss counts to `report`. Synchronises."""
        assert t.dtype == torch.bfloat16 and t.is_cuda and t.is_contiguous()
        self.call("dc_convert_bf16_to_f16", _stream(None), t.data_ptr(), t.data_ptr(), t.numel(),
                  ctypes.byref(report) if report is not None else None)
        return t.view(torch.float16)

    @property
    def launches(self) -> int:
        return int(self.lib.dc_launch_count(self.handle))

    @property
    def sm_count(self) -> int:
        return int(self.lib.dc_sm_count(self.handle))

    def reserve_workspace(self, nbytes: int):
        self.call("dc_reserve_workspace", nbytes)

    @staticmethod
    def tp_unique_id() -> bytes:
        """A fresh 128-byte id for a tensor-parallel group: make it on one rank, hand it to all."""
        lib = _lib.load()
        buf, err = ctypes.create_string_buffer(128), ctypes.create_string_buffer(256)
        rc = lib.dc_tp_unique_id(buf, err, len(err))
        if rc != 0:
            raise KernelError(rc, err.value.decode())
        return buf.raw

    def tp_init(self, unique_id: bytes, world: int, rank: int):
        """Joins this context to a tensor-parallel group (collective: every rank calls it with the same id)."""
        assert len(unique_id) == 128
        self.call("dc_tp_init", ctypes.create_string_buffer(unique_id, 128), world, rank)

    @property
    def tp_world(self) -> int:
        return int(self.lib.dc_tp_world(self.handle))

    @property
    def tp_rank(self) -> int:
        return int(self.lib.dc_tp_rank(self.handle))

    def tp_all_reduce_f32(self, t: torch.Tensor, stream=None):
        assert t.dtype == torch.float32 and t.is_cuda and t.is_contiguous()
        self.call("dc_tp_all_reduce_f32", _stream(stream), t.data_ptr(), t.numel())

    def set_workspace_frozen(self, on: bool):
        """Frozen: an op that needs more scratch than is reserved raises instead of reallocating the workspace."""
        self.call("dc_set_workspace_frozen", int(on))

    def warm_up(self):
        """Makes every kernel variant launchable now (Gemm::warm_up, kernels/gemm.rs:89-107)."""
        self.call("dc_warm_up")

    @property
    def workspace_bytes(self) -> int:
        return int(self.lib.dc_workspace_bytes(self.handle))

    @property
    def alloc_count(self) -> int:
        """Device/pinned allocations this context has made so far."""
        return int(self.lib.dc_alloc_count(self.handle))

    @property
    def tmap_encodes(self) -> int:
        """Tensor maps encoded so far (cache misses)."""
        return int(self.lib.dc_tmap_encode_count(self.handle))

    @property
    def tmap_cache_size(self) -> int:
        return int(self.lib.dc_tmap_cache_size(self.handle))


class _Family:
    def __init__(self, dev: Device):
        self.dev = dev


class Gemm(_Family):
    def implementation(self) -> Impl:
        return self.dev.get_impl(Family.Gemm)

    def gemm(self, stream, x, w, y, m, n, k, ldx, ldw, ldy, epi: Epilogue, swiglu_block: int = 16):
        """Y = X·Wᵀ then `epi` (kernels/gemm.rs:138-175)."""
        self.dev.call("dc_gemm", _stream(stream), _ptr(x), _ptr(w), _ptr(y), m, n, k, ldx, ldw, ldy, int(epi), swiglu_block)

    def gemm_tile(self, stream, x, w, y, m, n, k, ldx, ldw, ldy, epi: Epilogue, bn: int):
        """The fast kernel with a forced tile width (test hook)."""
        self.dev.call("dc_gemm_tile", _stream(stream), _ptr(x), _ptr(w), _ptr(y), m, n, k, ldx, ldw, ldy, int(epi), bn)

    def plan(self, m: int, n: int) -> int:
        return int(self.dev.lib.dc_gemm_plan(self.dev.handle, m, n))

    def plan_k(self, m: int, n: int, k: int) -> tuple[int, int]:
        """(tile width, K split of the tail wave's tiles) the fast GEMM uses for this shape."""
        split = ctypes.c_uint32(0)
        bn = int(self.dev.lib.dc_gemm_plan_k(self.dev.handle, m, n, k, ctypes.byref(split)))
        return bn, int(split.value)

    def plan_for(self, m: int, n: int, k: int, epi: Epilogue, bn: int = 0) -> tuple[int, int]:
        """(tile width, K split of the tail wave's tiles) for a shape and epilogue; bn forces the width (as gemm_tile does)."""
        split = ctypes.c_uint32(0)
        got = int(self.dev.lib.dc_gemm_plan_for(self.dev.handle, m, n, k, int(epi), bn, ctypes.byref(split)))
        assert got != 0, f"tile width {bn} is not one the fast GEMM has"
        return got, int(split.value)


class Norm(_Family):
    def rmsnorm(self, stream, x, w, y, rowmap, rows, h, ld_in, ld_out, add_one: bool, eps: float = EPS):
        """y[r] = rmsnorm(x[rowmap[r]])·(w or 1+w) as bf16 (kernels/norm.rs:23-33). rowmap None = identity."""
        self.dev.call("dc_rmsnorm", _stream(stream), _ptr(x), _ptr(w), _ptr(y), _ptr(rowmap), rows, h, ld_in, ld_out, eps, int(add_one))


    def add_rmsnorm(self, stream, x, add, w, y, rows, h, add_one: bool = True, eps: float = EPS):
        """x[r] += add[r], then y[r] = rmsnorm(x[r]) (y None: only the add). `add` is fp32, or in the context's 16-bit type
        (the partial sums of a tensor-parallel group; the reference's Ane::add_partial + rmsnorm, kernels/ane.rs:23)."""
        name = "dc_add_rmsnorm" if add.dtype == torch.float32 else "dc_add16_rmsnorm"
        self.dev.call(name, _stream(stream), _ptr(x), _ptr(add), _ptr(w), _ptr(y), rows, h, eps, int(add_one))


class Embed(_Family):
    def embed(self, stream, ids, table, out, t, h):
        """out[t] = table[ids[t]] (bf16 → fp32) (kernels/embed.rs:16-22)."""
        self.dev.call("dc_embed", _stream(stream), _ptr(ids), _ptr(table), _ptr(out), t, h)


class GNorm(_Family):
    def gated_rmsnorm_silu(self, stream, o, z, w, y, t, ldz, nv: int, dv: int = 128, eps: float = EPS):
        """Per (row, value head) RMSNorm × SiLU(z) (kernels/gnorm.rs:19-31)."""
        self.dev.call("dc_gated_rmsnorm_silu", _stream(stream), _ptr(o), _ptr(z), _ptr(w), _ptr(y), t, nv, dv, ldz, eps)


class Head(_Family):
    def gather_rows_f32(self, stream, x, rowmap, out, rows, h):
        self.dev.call("dc_gather_rows_f32", _stream(stream), _ptr(x), _ptr(rowmap), _ptr(out), rows, h)

    def gather_rows_bf16(self, stream, x, rowmap, out, rows, h):
        self.dev.call("dc_gather_rows_bf16", _stream(stream), _ptr(x), _ptr(rowmap), _ptr(out), rows, h)

    def final_head(self, stream, x, w, table, cand, ncand, logits, rows, h, max_cand, eps: float = EPS):
        """Final norm + candidate-row logits (kernels/head.rs:47-60)."""
        self.dev.call("dc_final_head", _stream(stream), _ptr(x), _ptr(w), _ptr(table), _ptr(cand), _ptr(ncand), _ptr(logits), rows, h, max_cand, eps)


class Rope(_Family):
    def q_norm_rope(self, stream, pq, qw, inv_freq, qpos, qo, rows, ldq, nq: int, hd: int, rot: int, eps: float = EPS):
        """Head norm + RoPE of the q heads (kernels/rope.rs:26-37)."""
        self.dev.call("dc_q_norm_rope", _stream(stream), _ptr(pq), _ptr(qw), _ptr(inv_freq), _ptr(qpos), _ptr(qo), rows, ldq, nq, hd, rot, eps)

    def kv_norm_rope(self, stream, pkv, kw, inv_freq, kc, vc, rows, ldkv, kcol, vcol, pos0, cache_rows: int, nkv: int,
                     hd: int, rot: int, pos=None, eps: float = EPS):
        """Head norm + RoPE of the k heads into the K cache, v heads copied to the V cache (kernels/rope.rs:39-51).
        `pos` (u32 per row) switches to packed sequences: rotate for pos[r], write cache row r."""
        self.dev.call("dc_kv_norm_rope", _stream(stream), _ptr(pkv), _ptr(kw), _ptr(inv_freq), _ptr(kc), _ptr(vc), rows, ldkv,
                      kcol, vcol, pos0, _ptr(pos), cache_rows, nkv, hd, rot, eps)


class Attn(_Family):
    def implementation(self) -> Impl:
        return self.dev.get_impl(Family.Attn)

    def attention(self, stream, q, kc, vc, gate, qpos, y, rows, ldg, nq: int, nkv: int, hd: int = 128, seq_start=None,
                  n_seq: int = 1, max_len: int = 0):
        """Causal GQA attention with the optional sigmoid gate (kernels/attn.rs:81-118). The reference passes
        the fused projection `pq` and reads the gate at a fixed column; here `gate` is that column's address
        (`(p, col * 4)`), or None for no gate."""
        self.dev.call("dc_attention", _stream(stream), _ptr(q), _ptr(kc), _ptr(vc), _ptr(gate), _ptr(qpos), _ptr(y), rows, ldg, nq,
                      nkv, hd, _ptr(seq_start), n_seq, max_len)


    def attention_rows(self, stream, q, kc, vc, gate, qpos, kv_start, y, rows, ldg, nq: int, nkv: int, hd: int = 128):
        """The same for a few query rows scattered over the packed caches of a batch (the pruned last layer's call,
        forward.rs:1176-1178): row r attends cache rows kv_start[r] .. kv_start[r] + qpos[r]."""
        self.dev.call("dc_attention_rows", _stream(stream), _ptr(q), _ptr(kc), _ptr(vc), _ptr(gate), _ptr(qpos), _ptr(kv_start), _ptr(y),
                      rows, ldg, nq, nkv, hd)


class Conv(_Family):
    def conv_silu_l2(self, stream, p, prev, w, q, k, v, t, ldp, nk: int, nv: int, dk: int = 128, dv: int = 128,
                     seq_start=None, n_seq: int = 1, max_len: int = 0):
        """Depthwise causal conv + SiLU + per-head L2 norm (kernels/conv.rs:21-36)."""
        self.dev.call("dc_conv_silu_l2", _stream(stream), _ptr(p), _ptr(prev), _ptr(w), _ptr(q), _ptr(k), _ptr(v), t, ldp, nk, nv, dk, dv,
                      _ptr(seq_start), n_seq, max_len)

    def conv_state_update(self, stream, p, prev_in, prev_out, t, ldp, conv_dim: int):
        """The 3 raw rows that end the chunk (kernels/conv.rs:38-46)."""
        self.dev.call("dc_conv_state_update", _stream(stream), _ptr(p), _ptr(prev_in), _ptr(prev_out), t, ldp, conv_dim)


class Delta(_Family):
    def implementation(self) -> Impl:
        return self.dev.get_impl(Family.Delta)

    def gated_delta(self, stream, q, k, v, a, b, a_log, dt_bias, state_in, state_out, o, t, ldab, write_state: bool,
                    nk: int, nv: int, dk: int = 128, dv: int = 128, seq_start=None, n_seq: int = 1, max_len: int = 0):
        """The gated delta rule (kernels/delta.rs:53-100)."""
        self.dev.call("dc_gated_delta", _stream(stream), _ptr(q), _ptr(k), _ptr(v), _ptr(a), _ptr(b), _ptr(a_log), _ptr(dt_bias),
                      _ptr(state_in), _ptr(state_out), _ptr(o), t, ldab, int(write_state), nk, nv, dk, dv, _ptr(seq_start), n_seq, max_len)

    def conv_gated_delta_supported(self) -> bool:
        return bool(self.dev.lib.dc_conv_gated_delta_supported(self.dev.handle))

    def conv_gated_delta(self, stream, p, prev, w, a, b, a_log, dt_bias, state_in, state_out, o, t, ldp, write_state: bool,
                         nk: int, nv: int, dk: int = 128, dv: int = 128, seq_start=None, n_seq: int = 1, max_len: int = 0):
        """conv_silu_l2 + gated_delta in one call: q, k, v never reach memory (no single counterpart in the reference)."""
        self.dev.call("dc_conv_gated_delta", _stream(stream), _ptr(p), _ptr(prev), _ptr(w), _ptr(a), _ptr(b), _ptr(a_log), _ptr(dt_bias),
                      _ptr(state_in), _ptr(state_out), _ptr(o), t, ldp, int(write_state), nk, nv, dk, dv, _ptr(seq_start), n_seq, max_len)


class Kernels:
    """Every kernel family, as `Kernels::new(dev)` of the reference (kernels/mod.rs:54-66)."""

    def __init__(self, dev: Device):
        self.dev = dev
        self.embed = Embed(dev)
        self.norm = Norm(dev)
        self.gemm = Gemm(dev)
        self.gnorm = GNorm(dev)
        self.head = Head(dev)
        self.rope = Rope(dev)
        self.attn = Attn(dev)
        self.conv = Conv(dev)
        self.delta = Delta(dev)
