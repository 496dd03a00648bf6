"""The public entry: a prefill engine for one GPU.

`Engine(dims, state_dict)` converts checkpoint-layout tensors to the fused layouts, uploads them and
creates the C++ model (libdecide_cuda.so `dc_model_*`); `engine.logits(batch)` runs one batched
prefill from host buffers and returns the candidate logits. This is the slice of the reference's
`Engine`/`Forward` (crates/decide-engine/src/engine.rs:226-230, forward.rs:704-731) that the hot path
needs: token ids in, candidate-row logits out. torch holds the device memory of the weights; every
computation happens in the library.
"""
from __future__ import annotations

import ctypes

import numpy as np
import torch

from .kernels import Act, ConvertReport, Device, KernelError, _stream
from .synth import Batch
from .weights import LAYER_FIELDS, CDims, CLayerWeights, Dims, fuse_layer, tp_shard_layer


def _u32p(a: np.ndarray):
    assert a.dtype == np.uint32 and a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(ctypes.c_void_p)


class Engine:
    def __init__(self, dims: Dims, state_dict: dict | None = None, dev: Device | None = None, max_rows: int = 4096,
                 max_seqs: int = 64, max_answers: int = 1024, max_cand: int = 16, fused_layers: list | None = None,
                 embed: torch.Tensor | None = None, final_norm: torch.Tensor | None = None):
        """Either `state_dict` (checkpoint names, CPU tensors) or already fused device tensors
        (`fused_layers`, `embed`, `final_norm`) must be given. `dims` are the WHOLE model's. When the device's
        context belongs to a tensor-parallel group (`Device.tp_init`), this engine is that rank's shard: a state
        dict is cut by `weights.tp_shard_layer`; fused layers given directly must already be the rank's slices."""
        self.dims = dims
        self.dev = dev or Device(0)
        self.tp_world, self.tp_rank = self.dev.tp_world, self.dev.tp_rank
        self.local_dims = dims.tp_local(self.tp_world) if self.tp_world > 1 else dims
        self.lib = self.dev.lib
        self.max_cand = max_cand
        cuda = torch.device("cuda", self.dev.device)
        if fused_layers is None:
            fused_layers = []
            for l in range(dims.n_layers):
                lw = fuse_layer(state_dict, l, dims)
                if self.tp_world > 1:
                    lw = tp_shard_layer(lw, l, dims, self.tp_world, self.tp_rank)
                fused_layers.append({k: v.to(cuda) for k, v in lw.items()})
            embed = state_dict["embed_tokens.weight"].to(torch.bfloat16).to(cuda)
            final_norm = state_dict["norm.weight"].to(torch.float32).to(cuda)
        # Weight matrices are stored in the context's 16-bit type. In fp16 mode the bf16 checkpoint values
        # are converted once, in place, refusing a model whose weights overflow fp16
        # (crates/decide-engine/src/convert.rs:73-98).
        self.convert_report = ConvertReport()
        if self.dev.act == Act.F16:
            for lw in fused_layers:
                for name in ("w_in", "w_out", "w_gu", "w_down"):
                    if lw[name].dtype == torch.bfloat16:
                        lw[name] = self.dev.convert_bf16_to_f16(lw[name], self.convert_report)
            if self.convert_report.f16_overflow:
                raise ValueError(f"{self.convert_report.f16_overflow} weights overflow fp16")
        want = torch.float16 if self.dev.act == Act.F16 else torch.bfloat16
        assert all(lw[n].dtype == want for lw in fused_layers for n in ("w_in", "w_out", "w_gu", "w_down")), "weights are not in the context's 16-bit type"
        self.layers, self.embed, self.final_norm = fused_layers, embed, final_norm  # keep the device tensors alive
        arr = (CLayerWeights * dims.n_layers)()
        for l, lw in enumerate(fused_layers):
            for name in LAYER_FIELDS:
                setattr(arr[l], name, lw[name].data_ptr() if name in lw else None)
        cd = CDims.of(self.local_dims)
        self.handle = self.lib.dc_model_create(self.dev.handle, ctypes.byref(cd), arr, embed.data_ptr(), final_norm.data_ptr(),
                                               max_rows, max_seqs, max_answers, max_cand)
        if not self.handle:
            raise KernelError(1, self.dev.last_error())

    def close(self):
        if getattr(self, "handle", None):
            self.lib.dc_model_destroy(self.handle)
            self.handle = None

    def _call(self, name, *args):
        rc = getattr(self.lib, name)(self.handle, *args)
        if rc != 0:
            raise KernelError(rc, self.dev.last_error())

    def logits(self, batch: Batch, stream=None) -> np.ndarray:
        """One batched prefill from host buffers: returns fp32 logits [n_ans, max_cand] (synchronous)."""
        n_ans = len(batch.ans_rows)
        out = np.zeros((n_ans, self.max_cand), dtype=np.float32)
        assert batch.cand.shape == (n_ans, self.max_cand)
        self._call("dc_model_prefill", _stream(stream), _u32p(batch.ids), _u32p(batch.seq_start), batch.n_seq, _u32p(batch.ans_rows),
                   _u32p(batch.cand), _u32p(batch.ncand), n_ans, out.ctypes.data_as(ctypes.c_void_p))
        return out

    def forward_resident(self, batch: Batch, stream=None):
        """Enqueues the same pass over the inputs the last `logits(batch)` left on the device."""
        self._call("dc_model_forward_resident", _stream(stream), _u32p(batch.seq_start), batch.n_seq, len(batch.ans_rows))

    def set_pruning(self, on: bool):
        """Last-layer pruning to the answer rows (Forward::set_pruning, forward.rs:517-522); on by default."""
        self._call("dc_model_set_pruning", int(on))

    def set_truncation(self, on: bool):
        """Stop each request after its last answer row (forward.rs:830-831); on by default."""
        self._call("dc_model_set_truncation", int(on))

    def set_graphs(self, on: bool):
        """Replay batched forwards of a shape seen before from a CUDA graph (default on)."""
        self._call("dc_model_set_graphs", int(on))

    @property
    def graph_count(self) -> int:
        return int(self.lib.dc_model_graph_count(self.handle))

    def set_chunk(self, rows: int):
        """A single request runs in chunks of at most `rows` rows with carried state (Forward::set_chunk, forward.rs:504-510); 0 = whole."""
        self._call("dc_model_set_chunk", rows)

    def build_snapshot(self, prefix_ids, stream=None):
        """Runs the constant prefix once and keeps the state after it (Forward::build_snapshot, forward.rs:645-673); later
        single requests that begin with these ids skip them. An empty prefix drops the snapshot."""
        ids = np.ascontiguousarray(prefix_ids, dtype=np.uint32)
        self._call("dc_model_build_snapshot", _stream(stream), _u32p(ids) if len(ids) else None, len(ids))

    @property
    def last_route(self) -> str:
        """How the last `logits` call ran its request (Route, forward.rs:196-206)."""
        return ("full", "snapshot", "state_cache")[int(self.lib.dc_model_last_route(self.handle))]

    @property
    def last_start(self) -> int:
        """The first row the last `logits` call computed (Forward::last_start, forward.rs:686-692)."""
        return int(self.lib.dc_model_last_start(self.handle))

    def set_state_cache(self, entries: int):
        """Hold up to `entries` (at most 4) states for follow-up questions; 0 turns the cache off
        (Forward::set_state_cache, forward.rs:735-744)."""
        self._call("dc_model_set_state_cache", entries)

    def forget_states(self):
        """Forget every cached state, keeping the buffers (Forward::forget_states, forward.rs:746-752)."""
        self.lib.dc_model_forget_states(self.handle)

    @property
    def state_cache_capacity(self) -> int:
        return int(self.lib.dc_model_state_cache_capacity(self.handle))

    def cached_states(self) -> list[int]:
        """Length in tokens of each cached state, most recently used first (Forward::cached_states, forward.rs:759-763)."""
        lens = np.zeros(4, dtype=np.uint32)
        n = int(self.lib.dc_model_cached_states(self.handle, _u32p(lens), 4))
        return [int(v) for v in lens[:n]]

    def set_state_marker(self, marker_ids):
        """The token ids that end a request's state; empties the cache (Forward::set_state_marker, forward.rs:765-772)."""
        ids = np.ascontiguousarray(marker_ids, dtype=np.uint32)
        self._call("dc_model_set_state_marker", _u32p(ids) if len(ids) else None, len(ids))

    @property
    def resident_rows(self) -> int:
        """Rows the last `logits` call ran after truncation."""
        return int(self.lib.dc_model_resident_rows(self.handle))

    def set_layer_limit(self, n: int):
        self._call("dc_model_set_layer_limit", n)

    def buffer(self, name: str, shape, dtype=np.float32) -> np.ndarray:
        """A host copy of a named activation buffer's leading elements (per-layer parity checks)."""
        out = np.empty(shape, dtype=dtype)
        self._call("dc_model_read_buffer", name.encode(), out.ctypes.data_as(ctypes.c_void_p), out.nbytes)
        return out

    def set_profiling(self, on: bool):
        self._call("dc_model_set_profiling", int(on))

    def profile(self) -> list[tuple[str, float, int]]:
        buf = ctypes.create_string_buffer(8192)
        self.lib.dc_model_profile(self.handle, buf, len(buf))
        rows = []
        for line in buf.value.decode().splitlines():
            name, ms, calls = line.split()
            rows.append((name, float(ms), int(calls)))
        return rows

    @property
    def activation_bytes(self) -> int:
        return int(self.lib.dc_model_activation_bytes(self.handle))
