"""Safetensors reading and writing, the manifest check and random weights."""
import json
import os
import struct

import numpy as np
import pytest
import torch

import tiny_configs
from crane_b200.parts import model_manifest
from crane_b200.config import HunyuanDenseConfig, build_spec
from crane_b200.weights import (DictSource, SafetensorsError, SafetensorsFile, TensorSpec,
                                WeightsError, load_weights, model_files, open_folder, save_file)
from crane_b200.weights.random_init import random_tensors, write_model_folder


def _manifest(cfg):
    return model_manifest(build_spec(HunyuanDenseConfig.from_dict(cfg)))


def test_round_trip_against_the_safetensors_library(tmp_path):
    from safetensors.torch import load_file, save_file as lib_save
    t = {"a.weight": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16),
         "idx": torch.arange(6, dtype=torch.int64).view(2, 3), "empty": torch.zeros(0, 4)}
    ours = str(tmp_path / "ours.safetensors")
    save_file(t, ours, {"k": "v"})
    back = load_file(ours)                                   # the library reads our file
    assert set(back) == set(t) and all(torch.equal(back[k], t[k]) for k in t)
    theirs = str(tmp_path / "theirs.safetensors")
    lib_save(t, theirs)
    f = SafetensorsFile(theirs)                              # we read the library's file
    assert sorted(f.names()) == sorted(t)
    for k in t:
        assert f.info(k) == (t[k].dtype, tuple(t[k].shape)) and torch.equal(f.tensor(k), t[k])


def test_truncated_and_broken_files(tmp_path):
    p = tmp_path / "model.safetensors"
    save_file({"w": torch.ones(4, 4)}, str(p))
    raw = p.read_bytes()
    p.write_bytes(raw[:-8])
    with pytest.raises(SafetensorsError, match="truncated"):
        SafetensorsFile(str(p))
    p.write_bytes(raw[:4])
    with pytest.raises(SafetensorsError, match="truncated"):
        SafetensorsFile(str(p))
    p.write_bytes(struct.pack("<Q", 10) + b"{not json}" + b"\0" * 8)
    with pytest.raises(SafetensorsError, match="not JSON"):
        SafetensorsFile(str(p))


def test_model_file_discovery(tmp_path):
    # crane-core/src/utils/utils.rs:16-57
    with pytest.raises(SafetensorsError, match="No valid model files"):
        model_files(str(tmp_path))
    save_file({"a": torch.ones(1)}, str(tmp_path / "model-00001-of-00002.safetensors"))
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(
        {"weight_map": {"a": "model-00001-of-00002.safetensors", "b": "model-00002-of-00002.safetensors"}}))
    with pytest.raises(SafetensorsError, match="Missing shard file"):
        model_files(str(tmp_path))
    save_file({"b": torch.ones(2)}, str(tmp_path / "model-00002-of-00002.safetensors"))
    assert len(model_files(str(tmp_path))) == 2
    src = open_folder(str(tmp_path))
    assert sorted(src.names()) == ["a", "b"] and src.tensor("b").shape == (2,)


def test_one_error_lists_missing_unexpected_and_wrong_shapes():
    man = _manifest(tiny_configs.A)
    t = random_tensors(man, 0, torch.float32)
    del t["model.norm.weight"], t["model.layers.1.mlp.up_proj.weight"]
    t["model.layers.0.self_attn.rotary.inv_freq"] = torch.zeros(8)
    t["model.layers.0.mlp.down_proj.weight"] = torch.zeros(64, 127)
    with pytest.raises(WeightsError) as e:
        load_weights(DictSource(t), man, {}, torch.float32, "cpu", "a test")
    msg = str(e.value)
    assert e.value.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert e.value.unexpected == ["model.layers.0.self_attn.rotary.inv_freq"]
    assert e.value.wrong == [("model.layers.0.mlp.down_proj.weight", (64, 128), (64, 127))]
    for word in ("missing tensors (2)", "unexpected tensors (1)", "wrong shapes (1)", "[64, 128]", "[64, 127]"):
        assert word in msg


def test_ignored_tensors_are_not_unexpected():
    cfg = HunyuanDenseConfig.from_dict(tiny_configs.A)
    spec = build_spec(cfg)
    man = model_manifest(spec)
    assert "lm_head.weight" not in man                     # tied
    t = random_tensors(man, 0, torch.float32)
    t["lm_head.weight"] = torch.zeros(256, 64)
    load_weights(DictSource(t), man, spec.ignored_tensors, torch.float32, "cpu")


def test_dtype_policy():
    man = {"m": TensorSpec((2, 2)), "n": TensorSpec((2,), "float32"), "k32": TensorSpec((2,), "keep"),
           "k16": TensorSpec((2,), "keep"), "tab": TensorSpec((3,), "keep")}
    t = {"m": torch.ones(2, 2), "n": torch.ones(2).bfloat16(), "k32": torch.ones(2),
         "k16": torch.ones(2).bfloat16(), "tab": torch.arange(3, dtype=torch.int64)}
    w = load_weights(DictSource(t), man, {}, torch.bfloat16, "cpu")
    assert w["m"].dtype == torch.bfloat16          # matrices in the model dtype
    assert w["n"].dtype == torch.float32           # norm weights always 32-bit
    assert w["k32"].dtype == torch.float32         # stored in 32-bit: stays so
    assert w["k16"].dtype == torch.bfloat16
    assert w["tab"].dtype == torch.int32           # integer tables
    assert load_weights(DictSource(t), man, {}, torch.float32, "cpu")["m"].dtype == torch.float32


def test_manifest_names_and_shapes():
    man = _manifest(tiny_configs.B)
    assert man["model.embed_tokens.weight"].shape == (384, 160)
    assert man["lm_head.weight"].shape == (384, 160)
    assert man["model.layers.2.self_attn.q_proj.weight"].shape == (256, 160)
    assert man["model.layers.2.self_attn.k_proj.weight"].shape == (64, 160)
    assert man["model.layers.2.self_attn.o_proj.weight"].shape == (160, 256)
    assert man["model.layers.0.mlp.gate_proj.weight"].shape == (352, 160)
    assert man["model.layers.0.mlp.down_proj.weight"].shape == (160, 352)
    assert not any("layernorm" in n and "self_attn" in n for n in man)       # qk norm off
    c = _manifest(tiny_configs.C)
    assert "model.layers.0.self_attn.q_proj.bias" in c and "model.layers.1.self_attn.k_proj.weight" not in c
    assert c["model.layers.1.self_attn.query_layernorm.weight"].shape == (48,)


def test_random_weights_are_seeded_and_independent_of_order(tmp_path):
    man = _manifest(tiny_configs.A)
    a, b = random_tensors(man, 5, torch.float32), random_tensors(man, 5, torch.float32)
    c = random_tensors(man, 6, torch.float32)
    assert all(torch.equal(a[k], b[k]) for k in a)
    assert not torch.equal(a["model.norm.weight"], c["model.norm.weight"])
    sub = {k: man[k] for k in list(man)[:3]}
    s = random_tensors(sub, 5, torch.float32)
    assert all(torch.equal(s[k], a[k]) for k in s)
    assert abs(float(a["model.norm.weight"].mean()) - 1.0) < 0.05
    assert 0.015 < float(a["model.embed_tokens.weight"].std()) < 0.025


def test_write_model_folder(tmp_path):
    d = write_model_folder(str(tmp_path / "m"), tiny_configs.B, 1, "bfloat16")
    assert sorted(os.listdir(d)) == ["config.json", "model.safetensors"]
    src = open_folder(d)
    man = _manifest(tiny_configs.B)
    assert set(src.names()) == set(man)
    assert src.info("model.layers.0.mlp.up_proj.weight")[0] == torch.bfloat16
    assert src.info("model.norm.weight")[0] == torch.float32
    assert json.load(open(os.path.join(d, "config.json")))["hidden_size"] == 160


def test_random_weights_command_line_writes_the_same_folder(tmp_path):
    from crane_b200.weights.random_init import main
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps(tiny_configs.A))
    assert main(["--config", str(cfg), "--out", str(tmp_path / "cli"), "--seed", "9"]) == 0
    write_model_folder(str(tmp_path / "api"), tiny_configs.A, 9, "bfloat16")
    a, b = open_folder(str(tmp_path / "cli")), open_folder(str(tmp_path / "api"))
    assert sorted(a.names()) == sorted(b.names())
    assert all(torch.equal(a.tensor(n), b.tensor(n)) for n in a.names())
