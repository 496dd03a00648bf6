"""The on-disk weight format `decide-weights-v1`: converter and loader.

Restates the reference's converter and loader for this engine
(crates/decide-engine/src/convert.rs:21-29, 94-197, 204-245, 296-395; weights.rs:15-50, 96-183):

  * a directory of blobs: `decide-embed.bin` (the bf16 embedding table alone) and `decide-lNN.bin`
    (8 layers each, NN = first layer), every tensor at a 16 KiB-aligned offset, the tail padded to
    16 KiB, little-endian;
  * `decide-index.json`: {"format": "decide-weights-v1", "blobs": [...], "tensors": {name:
    {"blob", "offset", "dtype", "shape"}}, "report": {...}} with tensor names `embed`,
    `L{i}.in_norm | w_in | q_norm | k_norm | conv_w | a_log | dt_bias | gnorm | w_out | post_norm |
    w_gu | w_down`, `final_norm`, written in forward-pass order;
  * projection matrices converted bf16 -> fp16 (round to nearest even) with the precision-loss
    report; any fp16 overflow fails the conversion and no index is written;
  * atomic commit: everything goes to `<name>.tmp`, the old index is removed first, blobs are
    renamed into place and the index last, so a directory is never half-loadable and a failed run
    leaves the previous conversion intact.

Two things differ from the reference, both because its model dims are compile-time constants and
this engine's are not: the index also carries a `"dims"` object (what config.json's check is for
the reference, config.rs:48-85), and the matrices may be kept as bf16 (`sixteen_bit="bf16"`) for a
bf16 context. The b and a blocks of a Gated DeltaNet in-projection are 16 rows each (zero rows past
the head count), identical to the reference's layout whenever the head count is a multiple of 16.

Sources: a state dict with the checkpoint's tensor names (what `decide_b200.synth` produces), or a
Hugging Face checkpoint directory (`model.safetensors.index.json` + shards, names under
`model.language_model.`), read with the `safetensors` package.
"""
from __future__ import annotations

import json
import mmap
import os
from dataclasses import asdict
from pathlib import Path

import numpy as np
import torch

from .weights import Dims, fuse_layer

ALIGN = 16 * 1024
INDEX_FILE = "decide-index.json"
FORMAT = "decide-weights-v1"
EMBED_BLOB = "decide-embed.bin"
LAYERS_PER_BLOB = 8
SRC_PREFIX = "model.language_model."
_SIZES = {"f16": 2, "bf16": 2, "f32": 4}
_TORCH = {"f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.float32}
LAYER_ORDER_ATTN = ("in_norm", "w_in", "q_norm", "k_norm", "w_out", "post_norm", "w_gu", "w_down")
LAYER_ORDER_GDN = ("in_norm", "w_in", "conv_w", "a_log", "dt_bias", "gnorm", "w_out", "post_norm", "w_gu", "w_down")


class ConvertError(RuntimeError):
    pass


def bf16_to_f16(t: torch.Tensor, report: dict) -> torch.Tensor:
    """bf16 -> fp16, round to nearest even, counting precision loss as convert.rs:73-90 does."""
    assert t.dtype == torch.bfloat16
    x = t.float()
    h = x.to(torch.float16)
    mag = h.view(torch.int16).to(torch.int32) & 0x7FFF
    report["f16_values"] += x.numel()
    over = (mag == 0x7C00) & torch.isfinite(x)
    flushed = (mag == 0) & (x != 0)
    sub = (mag != 0) & (mag < 0x0400)
    report["f16_overflow"] += int(over.sum())
    report["f16_flushed_to_zero"] += int(flushed.sum())
    report["f16_subnormal"] += int(sub.sum())
    return h


def _bytes_of(t: torch.Tensor) -> bytes:
    t = t.contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().tobytes()
    return t.numpy().tobytes()


class _Blob:
    """One output blob, written to `<name>.tmp` until commit (convert.rs:358-395)."""

    def __init__(self, out_dir: Path, name: str):
        self.name, self.path, self.tmp = name, out_dir / name, out_dir / (name + ".tmp")
        self.file = open(self.tmp, "wb")
        self.len = 0
        self.committed = False

    def _pad(self):
        pad = -self.len % ALIGN
        if pad:
            self.file.write(b"\0" * pad)
            self.len += pad

    def put(self, data: bytes) -> int:
        self._pad()
        offset = self.len
        self.file.write(data)
        self.len += len(data)
        return offset

    def commit(self):
        self._pad()
        self.file.flush()
        os.fsync(self.file.fileno())
        self.file.close()
        os.replace(self.tmp, self.path)
        self.committed = True

    def discard(self):
        if not self.committed:
            try:
                self.file.close()
                self.tmp.unlink()
            except OSError:
                pass


def _write_then_rename(path: Path, data: bytes):
    tmp = path.with_name(path.name + ".tmp")
    with open(tmp, "wb") as f:
        f.write(data)
        f.flush()
        os.fsync(f.fileno())
    os.replace(tmp, path)


def convert_state_dict(sd: dict, dims: Dims, out_dir, sixteen_bit: str = "f16") -> dict:
    """Writes `sd` (checkpoint names, bf16 projections) as a decide-weights-v1 directory. Returns the report.
    Raises ConvertError, leaving any previous conversion in `out_dir` intact, if a weight overflows fp16."""
    assert sixteen_bit in ("f16", "bf16")
    out_dir = Path(out_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    blob_names = [EMBED_BLOB] + [f"decide-l{l:02d}.bin" for l in range(0, dims.n_layers, LAYERS_PER_BLOB)]
    blobs = [_Blob(out_dir, n) for n in blob_names]
    tensors: dict = {}
    report = {"tensors": 0, "f16_values": 0, "f16_subnormal": 0, "f16_flushed_to_zero": 0, "f16_overflow": 0}
    overflowed: list[str] = []

    def put(blob: int, name: str, t: torch.Tensor):
        if name in tensors:
            raise ConvertError(f"tensor {name} written twice")
        if t.dtype == torch.bfloat16 and name != "embed" and sixteen_bit == "f16":
            before = report["f16_overflow"]
            t = bf16_to_f16(t, report)
            if report["f16_overflow"] > before:
                overflowed.append(name)
        dtype = {torch.float16: "f16", torch.bfloat16: "bf16", torch.float32: "f32"}[t.dtype]
        offset = blobs[blob].put(_bytes_of(t))
        tensors[name] = {"blob": blobs[blob].name, "offset": offset, "dtype": dtype, "shape": list(t.shape)}
        report["tensors"] += 1

    try:
        embed = sd["embed_tokens.weight"]
        if embed.dtype != torch.bfloat16 or tuple(embed.shape) != (dims.vocab, dims.hidden):
            raise ConvertError(f"embed_tokens.weight is {embed.dtype} {tuple(embed.shape)}; expected bf16 {(dims.vocab, dims.hidden)}")
        put(0, "embed", embed)
        for l in range(dims.n_layers):
            lw = fuse_layer(sd, l, dims)
            for field in (LAYER_ORDER_ATTN if dims.is_full_attention(l) else LAYER_ORDER_GDN):
                put(1 + l // LAYERS_PER_BLOB, f"L{l}.{field}", lw[field])
        put(len(blobs) - 1, "final_norm", sd["norm.weight"].to(torch.float32))
        if report["f16_overflow"]:
            raise ConvertError(f"{report['f16_overflow']} weights overflow fp16 (in {', '.join(overflowed)}); no index written")
        # Commit. The old index goes first: until the new one lands the directory must not look loadable.
        index_file = out_dir / INDEX_FILE
        try:
            index_file.unlink()
        except FileNotFoundError:
            pass
        for b in blobs:
            b.commit()
        index = {"format": FORMAT, "blobs": blob_names, "tensors": tensors, "report": report,
                 "dims": {k: (bool(v) if isinstance(v, bool) else v) for k, v in asdict(dims).items()}}
        _write_then_rename(index_file, json.dumps(index, indent=2).encode())
        return report
    finally:
        for b in blobs:
            b.discard()


def read_checkpoint(model_dir) -> tuple[dict, Dims]:
    """A Hugging Face checkpoint directory -> (state dict with names relative to `model.language_model.`, dims read
    from config.json's text_config). Only language-model tensors are read (the vision tower's are skipped, convert.rs:119-135)."""
    from safetensors import safe_open

    model_dir = Path(model_dir)
    cfg = json.loads((model_dir / "config.json").read_text())
    tc = cfg.get("text_config", cfg)
    rope = tc.get("rope_parameters") or {}
    dims = Dims(hidden=tc["hidden_size"], n_layers=tc["num_hidden_layers"], nq=tc["num_attention_heads"], nkv=tc["num_key_value_heads"],
                head_dim=tc["head_dim"], rot_dim=int(tc["head_dim"] * rope.get("partial_rotary_factor", tc.get("partial_rotary_factor", 1.0))),
                gdn_nk=tc["linear_num_key_heads"], gdn_nv=tc["linear_num_value_heads"], gdn_dk=tc["linear_key_head_dim"],
                gdn_dv=tc["linear_value_head_dim"], inter=tc["intermediate_size"], vocab=tc["vocab_size"],
                full_attn_interval=tc.get("full_attention_interval", 4), attn_gate=bool(tc.get("attn_output_gate", True)),
                eps=tc.get("rms_norm_eps", 1e-6), rope_theta=float(rope.get("rope_theta", tc.get("rope_theta", 1e7))))
    weight_map = json.loads((model_dir / "model.safetensors.index.json").read_text())["weight_map"]
    sd = {}
    by_file: dict[str, list[str]] = {}
    for name, file in weight_map.items():
        if name.startswith(SRC_PREFIX):
            by_file.setdefault(file, []).append(name)
    for file, names in by_file.items():
        with safe_open(str(model_dir / file), framework="pt") as f:
            for name in names:
                sd[name[len(SRC_PREFIX):]] = f.get_tensor(name)
    return sd, dims


def convert_checkpoint(model_dir, out_dir, sixteen_bit: str = "f16") -> dict:
    """`decide convert`: a Hugging Face checkpoint directory -> decide-weights-v1 in `out_dir` (which must differ)."""
    if Path(model_dir).resolve() == Path(out_dir).resolve():
        raise ConvertError("--out must differ from the model directory")
    sd, dims = read_checkpoint(model_dir)
    return convert_state_dict(sd, dims, out_dir, sixteen_bit)


class Weights:
    """A converted weights directory, blobs mapped read-only (weights.rs:96-183). `tensor(name)` gives a CPU torch
    tensor that aliases the mapping; `to_device` uploads a layer's tensors."""

    def __init__(self, directory):
        self.dir = Path(directory)
        index_path = self.dir / INDEX_FILE
        if not index_path.exists():
            raise FileNotFoundError(f"{index_path} does not exist; run the converter")
        index = json.loads(index_path.read_text())
        if index.get("format") != FORMAT:
            raise ValueError(f"{index_path} has format {index.get('format')!r}; expected {FORMAT}")
        self.dims = Dims(**index["dims"])
        self.report = index.get("report", {})
        self._maps, self._files = {}, []
        for name in index["blobs"]:
            f = open(self.dir / name, "rb")
            self._files.append(f)
            self._maps[name] = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
        self.entries = {}
        for name, e in index["tensors"].items():
            blob, offset, dtype, shape = e["blob"], int(e["offset"]), e["dtype"], [int(s) for s in e["shape"]]
            if blob not in self._maps:
                raise ValueError(f"tensor {name} is in {blob}, which is not in the blob list")
            if dtype not in _SIZES:
                raise ValueError(f"tensor {name}: unknown dtype {dtype!r}")
            if offset % ALIGN:
                raise ValueError(f"tensor {name}: offset {offset} is not {ALIGN}-byte aligned")
            nbytes = _SIZES[dtype] * int(np.prod(shape, dtype=np.int64))
            if offset + nbytes > len(self._maps[blob]):
                raise ValueError(f"tensor {name} runs past the end of {blob}")
            self.entries[name] = (blob, offset, dtype, shape, nbytes)

    def tensor(self, name: str) -> torch.Tensor:
        blob, offset, dtype, shape, nbytes = self.entries[name]
        raw = np.frombuffer(self._maps[blob], dtype=np.uint8, count=nbytes, offset=offset)
        import warnings

        with warnings.catch_warnings():
            warnings.simplefilter("ignore")   # the mapping is read-only; the tensors are only ever read
            t = torch.from_numpy(raw)
        return t.view(_TORCH[dtype]).reshape(shape)

    def sixteen_bit(self) -> str:
        return self.entries["L0.w_in"][2]

    def layer(self, l: int, device=None) -> dict:
        fields = LAYER_ORDER_ATTN if self.dims.is_full_attention(l) else LAYER_ORDER_GDN
        return {f: (self.tensor(f"L{l}.{f}").to(device) if device is not None else self.tensor(f"L{l}.{f}")) for f in fields}

    def close(self):
        self.entries = {}
        for m in self._maps.values():
            try:
                m.close()
            except BufferError:
                pass   # a tensor still aliases the mapping; it is released with it
        for f in self._files:
            f.close()
        self._maps, self._files = {}, []


def open_engine(directory, dev=None, **engine_kw):
    """Engine::open's weight half (engine.rs:145-185): map a converted directory and upload it. The directory's
    16-bit type must be the context's (fp16 matrices for the default context)."""
    from .engine import Engine
    from .kernels import Act, Device

    dev = dev or Device(0)
    w = Weights(directory)
    want = "f16" if dev.act == Act.F16 else "bf16"
    if w.sixteen_bit() != want:
        raise ValueError(f"{directory} holds {w.sixteen_bit()} matrices but the context's 16-bit type is {want}")
    cuda = torch.device("cuda", dev.device)
    if dev.tp_world > 1:   # one rank of a tensor-parallel group uploads only its slices
        from .weights import tp_shard_layer

        layers = [{k: v.to(cuda) for k, v in tp_shard_layer(w.layer(l), l, w.dims, dev.tp_world, dev.tp_rank).items()} for l in range(w.dims.n_layers)]
    else:
        layers = [w.layer(l, cuda) for l in range(w.dims.n_layers)]
    eng = Engine(w.dims, dev=dev, fused_layers=layers, embed=w.tensor("embed").to(cuda), final_norm=w.tensor("final_norm").to(cuda), **engine_kw)
    w.close()
    return eng
