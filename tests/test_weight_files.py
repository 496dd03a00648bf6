"""The on-disk weight format (decide-weights-v1) on the CPU: layout rules of the reference's converter
(crates/decide-engine/src/convert.rs:21-29, 94-197, 296-395) and the checks of its loader
(weights.rs:96-183): 16 KiB alignment, blob naming, index contents, fp16 conversion report, refusal
of fp16 overflow with the previous conversion left intact, nothing half-written ever loadable."""
import json

import numpy as np
import pytest
import torch

from decide_b200 import weight_files as wf
from decide_b200.synth import synth_state_dict
from decide_b200.weights import Dims, fuse_layer

DIMS = Dims(hidden=64, n_layers=10, nq=2, nkv=1, head_dim=128, rot_dim=32, gdn_nk=2, gdn_nv=4, inter=96, vocab=40)


def test_layout_index_and_round_trip(tmp_path):
    sd = synth_state_dict(DIMS, seed=3)
    report = wf.convert_state_dict(sd, DIMS, tmp_path)
    index = json.loads((tmp_path / wf.INDEX_FILE).read_text())
    assert index["format"] == "decide-weights-v1"
    assert index["blobs"] == ["decide-embed.bin", "decide-l00.bin", "decide-l08.bin"]   # 8 layers per blob
    assert not list(tmp_path.glob("*.tmp"))
    for name in index["blobs"]:
        assert (tmp_path / name).stat().st_size % wf.ALIGN == 0                          # whole 16 KiB pages
    names = list(index["tensors"])
    assert names[0] == "embed" and names[-1] == "final_norm"
    assert names[1:11] == [f"L0.{f}" for f in wf.LAYER_ORDER_GDN]                        # forward-pass order
    assert index["tensors"]["L3.w_in"]["dtype"] == "f16" and index["tensors"]["embed"]["dtype"] == "bf16"
    assert index["tensors"]["final_norm"]["blob"] == "decide-l08.bin"
    assert all(e["offset"] % wf.ALIGN == 0 for e in index["tensors"].values())
    assert report["tensors"] == len(names) and report["f16_overflow"] == 0

    w = wf.Weights(tmp_path)
    assert w.dims == DIMS and w.sixteen_bit() == "f16"
    assert torch.equal(w.tensor("embed"), sd["embed_tokens.weight"])
    values = 0
    for l in range(DIMS.n_layers):
        want = fuse_layer(sd, l, DIMS)
        got = w.layer(l)
        assert set(got) == set(want)
        for k, t in want.items():
            if t.dtype == torch.bfloat16:
                values += t.numel()
                assert torch.equal(got[k], t.float().to(torch.float16)), (l, k)
            else:
                assert torch.equal(got[k], t), (l, k)
    assert report["f16_values"] == values
    w.close()


def test_bf16_directory_keeps_the_bits(tmp_path):
    sd = synth_state_dict(DIMS, seed=4)
    wf.convert_state_dict(sd, DIMS, tmp_path, sixteen_bit="bf16")
    w = wf.Weights(tmp_path)
    assert w.sixteen_bit() == "bf16"
    assert torch.equal(w.tensor("L0.w_gu"), fuse_layer(sd, 0, DIMS)["w_gu"])
    w.close()


def test_precision_loss_report_counts():
    x = torch.tensor([1.0, 1e-5, -3e-6, 1e-9, 7e4, -1e30, 6.2e-5, 0.0, float("inf")]).to(torch.bfloat16)
    rep = {"f16_values": 0, "f16_subnormal": 0, "f16_flushed_to_zero": 0, "f16_overflow": 0}
    h = wf.bf16_to_f16(x, rep)
    assert rep == {"f16_values": 9, "f16_subnormal": 2, "f16_flushed_to_zero": 1, "f16_overflow": 2}
    assert torch.equal(h, x.float().to(torch.float16))


def test_overflow_fails_and_leaves_the_previous_conversion(tmp_path):
    sd = synth_state_dict(DIMS, seed=5)
    wf.convert_state_dict(sd, DIMS, tmp_path)
    before = (tmp_path / wf.INDEX_FILE).read_bytes(), (tmp_path / "decide-l00.bin").read_bytes()
    bad = dict(sd)
    bad["layers.2.mlp.down_proj.weight"] = sd["layers.2.mlp.down_proj.weight"].clone()
    bad["layers.2.mlp.down_proj.weight"][1, 1] = 1e6          # finite in bf16, infinite in fp16
    with pytest.raises(wf.ConvertError, match="overflow fp16.*L2.w_down"):
        wf.convert_state_dict(bad, DIMS, tmp_path)
    assert ((tmp_path / wf.INDEX_FILE).read_bytes(), (tmp_path / "decide-l00.bin").read_bytes()) == before
    assert not list(tmp_path.glob("*.tmp"))


def test_loader_refuses_what_the_reference_refuses(tmp_path):
    with pytest.raises(FileNotFoundError):
        wf.Weights(tmp_path)
    sd = synth_state_dict(DIMS, seed=6)
    wf.convert_state_dict(sd, DIMS, tmp_path)
    index = json.loads((tmp_path / wf.INDEX_FILE).read_text())
    for mutate, msg in [(lambda i: i.update(format="decide-weights-v0"), "format"),
                        (lambda i: i["tensors"]["L0.w_in"].update(offset=8), "aligned"),
                        (lambda i: i["tensors"]["L0.w_in"].update(offset=1 << 30), "past the end"),
                        (lambda i: i["tensors"]["L0.w_in"].update(blob="other.bin"), "blob list"),
                        (lambda i: i["tensors"]["L0.w_in"].update(dtype="f64"), "dtype")]:
        broken = json.loads(json.dumps(index))
        mutate(broken)
        (tmp_path / wf.INDEX_FILE).write_text(json.dumps(broken))
        with pytest.raises(ValueError, match=msg):
            wf.Weights(tmp_path)


def test_checkpoint_directory_is_read_by_prefix(tmp_path):
    """A Hugging Face directory: names under model.language_model., several shards, other towers skipped."""
    from safetensors.torch import save_file

    src, out = tmp_path / "hf", tmp_path / "out"
    src.mkdir()
    sd = synth_state_dict(DIMS, seed=7)
    names = sorted(sd)
    shards = {"a.safetensors": names[::2], "b.safetensors": names[1::2]}
    weight_map = {}
    for file, ns in shards.items():
        tensors = {wf.SRC_PREFIX + n: sd[n].contiguous() for n in ns}
        if file.startswith("a"):
            tensors["model.visual.patch_embed.weight"] = torch.zeros(4)
        save_file(tensors, str(src / file))
        weight_map.update({k: file for k in tensors})
    (src / "model.safetensors.index.json").write_text(json.dumps({"weight_map": weight_map}))
    (src / "config.json").write_text(json.dumps({"text_config": {
        "hidden_size": 64, "num_hidden_layers": 10, "num_attention_heads": 2, "num_key_value_heads": 1, "head_dim": 128,
        "linear_num_key_heads": 2, "linear_num_value_heads": 4, "linear_key_head_dim": 128, "linear_value_head_dim": 128,
        "intermediate_size": 96, "vocab_size": 40, "full_attention_interval": 4, "rms_norm_eps": 1e-6,
        "rope_parameters": {"rope_theta": 1e6, "partial_rotary_factor": 0.25}}}))
    got_sd, dims = wf.read_checkpoint(src)
    assert dims == DIMS and set(got_sd) == set(sd)
    wf.convert_checkpoint(src, out)
    w = wf.Weights(out)
    assert torch.equal(w.tensor("L9.w_down"), sd["layers.9.mlp.down_proj.weight"].float().to(torch.float16))
    w.close()
    with pytest.raises(wf.ConvertError):
        wf.convert_checkpoint(src, src)
