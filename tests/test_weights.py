"""Weights (no GPU): safetensors reading and writing, binding by name with ONE error that
lists missing and unexpected tensors and wrong shapes, kept types, random-weights mode."""
import json
import os
import struct

import pytest
import torch

from mormot2_ai_b200 import (DecoderModel, SafeTensorsFolder, WeightsError, write_random_model,
                             write_safetensors)
from mormot2_ai_b200.weights import bind_tensors, check_names, convert
from mormot2_ai_b200.weights.safetensors_file import SafeTensorsFile
from tests.conftest import tiny_a, tiny_b


def folder_tensors(folder):
    f = SafeTensorsFolder(folder)
    return {n: f.tensor(n).clone() for n in f.names()}


def rewrite(folder, tensors):
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors)


def needs_of(cfg):
    return DecoderModel(cfg.to_model_spec()).tensors()


def test_random_model_folder_is_complete_and_seeded(tmp_path):
    cfg = tiny_b()
    a = write_random_model(str(tmp_path / "a"), cfg, 1, std=0.03)
    b = write_random_model(str(tmp_path / "b"), cfg, 1, std=0.03)
    c = write_random_model(str(tmp_path / "c"), cfg, 2, std=0.03)
    ta, tb, tc = folder_tensors(a), folder_tensors(b), folder_tensors(c)
    check_names(needs_of(cfg), SafeTensorsFolder(a))
    assert set(ta) == {n.name for n in needs_of(cfg) if not n.optional}
    assert all(torch.equal(ta[n].view(torch.int16), tb[n].view(torch.int16)) for n in ta)
    assert any(not torch.equal(ta[n].view(torch.int16), tc[n].view(torch.int16)) for n in ta)
    assert all(t.dtype == torch.bfloat16 for t in ta.values())
    w = ta["model.layers.0.self_attn.q_proj.weight"].float()
    assert w.shape == (cfg.q_width, cfg.hidden_size) and abs(w.std().item() - 0.03) < 0.004
    n = ta["model.norm.weight"].float()
    assert abs(n.mean().item() - 1.0) < 0.05
    assert "lm_head.weight" in ta and "lm_head.weight" not in folder_tensors(
        write_random_model(str(tmp_path / "tied"), tiny_a(), 0))
    assert json.load(open(os.path.join(a, "config.json")))["architectures"] == ["Qwen3ForCausalLM"]


def test_one_error_lists_everything(tmp_path):
    cfg = tiny_a()
    folder = write_random_model(str(tmp_path / "m"), cfg, 0)
    t = folder_tensors(folder)
    del t["model.layers.1.mlp.up_proj.weight"]
    del t["model.norm.weight"]
    t["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    t["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(32, 64, dtype=torch.bfloat16)
    t["model.layers.1.input_layernorm.weight"] = torch.zeros(64, dtype=torch.float16)
    rewrite(folder, t)
    with pytest.raises(WeightsError) as e:
        bind_tensors(needs_of(cfg), SafeTensorsFolder(folder), torch.bfloat16, torch.device("cpu"))
    text = str(e.value)
    assert "missing (2)" in text and "model.layers.1.mlp.up_proj.weight" in text
    assert "model.norm.weight" in text
    assert "unexpected (1)" in text and "rotary_emb.inv_freq" in text
    assert "wrong shape (1)" in text and "[32, 64]" in text and "[64, 64]" in text
    assert "wrong type (1)" in text and "float16" in text


def test_kept_types(tmp_path):
    cfg = tiny_a()
    folder = write_random_model(str(tmp_path / "m"), cfg, 0)
    t = folder_tensors(folder)
    t["model.norm.weight"] = t["model.norm.weight"].float()       # stored in 32 bits
    rewrite(folder, t)
    cpu = torch.device("cpu")
    bf = bind_tensors(needs_of(cfg), SafeTensorsFolder(folder), torch.bfloat16, cpu)
    assert bf["model.norm.weight"].dtype == torch.float32          # stays so
    assert bf["model.embed_tokens.weight"].dtype == torch.bfloat16
    fp = bind_tensors(needs_of(cfg), SafeTensorsFolder(folder), torch.float32, cpu)
    assert all(v.dtype == torch.float32 for v in fp.values())
    assert torch.equal(fp["model.embed_tokens.weight"], bf["model.embed_tokens.weight"].float())
    assert convert(torch.tensor([1, 2], dtype=torch.int64), torch.bfloat16).dtype == torch.int32


def test_tied_head_stored_copy(tmp_path):
    cfg = tiny_a()
    folder = write_random_model(str(tmp_path / "m"), cfg, 0)
    t = folder_tensors(folder)
    t["lm_head.weight"] = t["model.embed_tokens.weight"].clone()
    rewrite(folder, t)
    out = bind_tensors(needs_of(cfg), SafeTensorsFolder(folder), torch.bfloat16, torch.device("cpu"))
    assert "lm_head.weight" not in out
    t["lm_head.weight"][3, 5] += 1.0
    rewrite(folder, t)
    with pytest.raises(WeightsError, match="tied"):
        bind_tensors(needs_of(cfg), SafeTensorsFolder(folder), torch.bfloat16, torch.device("cpu"))
    # untied without lm_head.weight
    folder_b = write_random_model(str(tmp_path / "b"), tiny_b(), 1)
    tb = folder_tensors(folder_b)
    del tb["lm_head.weight"]
    rewrite(folder_b, tb)
    with pytest.raises(WeightsError, match="lm_head.weight"):
        check_names(needs_of(tiny_b()), SafeTensorsFolder(folder_b))


def test_index_file(tmp_path):
    cfg = tiny_a()
    folder = write_random_model(str(tmp_path / "m"), cfg, 0)
    t = folder_tensors(folder)
    os.unlink(os.path.join(folder, "model.safetensors"))
    names = sorted(t)
    parts = {"model-00001-of-00002.safetensors": names[:10],
             "model-00002-of-00002.safetensors": names[10:]}
    weight_map = {}
    for fname, ns in parts.items():
        write_safetensors(os.path.join(folder, fname), {n: t[n] for n in ns})
        weight_map.update({n: fname for n in ns})
    index = os.path.join(folder, "model.safetensors.index.json")
    json.dump({"metadata": {}, "weight_map": weight_map}, open(index, "w"))
    f = SafeTensorsFolder(folder)
    assert f.names() == names
    assert torch.equal(f.tensor(names[12]).view(torch.int16), t[names[12]].view(torch.int16))
    del weight_map[names[0]]
    json.dump({"weight_map": weight_map}, open(index, "w"))
    with pytest.raises(WeightsError, match="index does not say so"):
        SafeTensorsFolder(folder)
    with pytest.raises(WeightsError, match="no model.safetensors"):
        SafeTensorsFolder(str(tmp_path))


def test_damaged_files(tmp_path):
    p = str(tmp_path / "x.safetensors")
    write_safetensors(p, {"a": torch.arange(6, dtype=torch.float32).reshape(2, 3),
                          "b": torch.ones(4, dtype=torch.bfloat16)})
    f = SafeTensorsFile(p)
    assert f.tensor("a").tolist() == [[0, 1, 2], [3, 4, 5]] and f.shape("b") == (4,)
    raw = open(p, "rb").read()
    open(p, "wb").write(raw[:-3])                      # cut short
    with pytest.raises(WeightsError):
        SafeTensorsFile(p)
    open(p, "wb").write(raw + b"\0\0")                 # trailing bytes
    with pytest.raises(WeightsError, match="after the last tensor"):
        SafeTensorsFile(p)
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n])
    header["a"]["shape"] = [2, 4]                      # shape and bytes disagree
    h = json.dumps(header).encode()
    open(p, "wb").write(struct.pack("<Q", len(h)) + h + raw[8 + n:])
    with pytest.raises(WeightsError, match="needs"):
        SafeTensorsFile(p)
    open(p, "wb").write(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(WeightsError, match="header"):
        SafeTensorsFile(p)
    dup = b'{"a":{"dtype":"F32","shape":[1],"data_offsets":[0,4]},"a":{"dtype":"F32","shape":[1],"data_offsets":[0,4]}}'
    open(p, "wb").write(struct.pack("<Q", len(dup)) + dup + b"\0\0\0\0")
    with pytest.raises(WeightsError, match="twice"):
        SafeTensorsFile(p)
