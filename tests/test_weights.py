"""Weights: the safetensors container, loading by name with one clear error, dtype policy, random-weights mode."""
import json
import os
import struct

import numpy as np
import pytest
import torch

from fusezap_core_b200.config import describe
from fusezap_core_b200.engine.model import declared_tensors, load_model
from fusezap_core_b200.weights import (SafetensorsError, WeightsError, read_file, read_model_dir, write_file,
                                       write_random_model)
from plain_ops import PlainOps
from tiny_configs import get
from util import make_model_dir, read_weights


def test_container_round_trip_against_the_safetensors_package(tmp_path):
    g = torch.Generator().manual_seed(0)
    t = {"a.weight": torch.randn(5, 7, generator=g), "b": torch.randn(3, generator=g).to(torch.bfloat16),
         "ids": torch.arange(6, dtype=torch.int64).view(2, 3), "h": torch.randn(4, generator=g).to(torch.float16)}
    fn = str(tmp_path / "x.safetensors")
    write_file(fn, t)
    from safetensors.torch import load_file, save_file
    theirs = load_file(fn)
    assert set(theirs) == set(t) and all(torch.equal(theirs[k], t[k]) and theirs[k].dtype == t[k].dtype for k in t)
    save_file(t, str(tmp_path / "y.safetensors"), metadata={"format": "pt"})
    mine = read_file(str(tmp_path / "y.safetensors"))
    assert set(mine) == set(t) and all(torch.equal(mine[k], t[k]) and mine[k].dtype == t[k].dtype for k in t)


def test_shards_and_index(tmp_path):
    a, b = {"x": torch.ones(2, 2)}, {"y": torch.zeros(3)}
    write_file(str(tmp_path / "model-00001-of-00002.safetensors"), a)
    write_file(str(tmp_path / "model-00002-of-00002.safetensors"), b)
    assert set(read_model_dir(str(tmp_path))) == {"x", "y"}
    with open(tmp_path / "model.safetensors.index.json", "w") as f:
        json.dump({"weight_map": {"x": "model-00001-of-00002.safetensors"}}, f)
    assert set(read_model_dir(str(tmp_path))) == {"x"}
    with open(tmp_path / "model.safetensors.index.json", "w") as f:
        json.dump({"weight_map": {"x": "gone.safetensors"}}, f)
    with pytest.raises(FileNotFoundError, match="gone.safetensors"):
        read_model_dir(str(tmp_path))
    os.makedirs(tmp_path / "empty")
    with pytest.raises(FileNotFoundError, match="no .safetensors"):
        read_model_dir(str(tmp_path / "empty"))


def test_corrupt_files(tmp_path):
    fn = str(tmp_path / "bad.safetensors")
    with open(fn, "wb") as f:
        f.write(b"\x01\x02")
    with pytest.raises(SafetensorsError, match="shorter"):
        read_file(fn)
    with open(fn, "wb") as f:
        f.write(struct.pack("<Q", 10 ** 9) + b"{}")
    with pytest.raises(SafetensorsError, match="header length"):
        read_file(fn)
    with open(fn, "wb") as f:
        f.write(struct.pack("<Q", 4) + b"nope")
    with pytest.raises(SafetensorsError, match="not JSON"):
        read_file(fn)
    hdr = json.dumps({"t": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}).encode()
    with open(fn, "wb") as f:
        f.write(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)   # truncated data
    with pytest.raises(SafetensorsError, match="spans bytes"):
        read_file(fn)


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    d, cfg, _ = make_model_dir("tiny_qwen2", tmp_path)
    w = read_weights(d)
    del w["model.layers.1.mlp.up_proj.weight"]
    del w["model.layers.2.self_attn.k_proj.bias"]                      # breaks an all-or-none group
    w["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(16)    # a buffer some exporters write: passed over
    w["model.layers.0.self_attn.extra_gate.weight"] = torch.zeros(16)
    w["model.norm.weight"] = torch.ones(97)
    write_file(os.path.join(d, "model.safetensors"), w)
    with pytest.raises(WeightsError) as e:
        load_model(d, "float32", "cpu", ops=PlainOps())
    msg = str(e.value)
    assert "model.layers.1.mlp.up_proj.weight" in msg and "model.layers.2.self_attn.k_proj.bias" in msg
    assert "extra_gate.weight" in msg and "rotary_emb.inv_freq" not in msg
    assert "model.norm.weight: shape (97,), expected (96,)" in msg
    assert e.value.missing and e.value.unexpected and e.value.wrong
    assert "missing (2)" in msg and "unexpected (1)" in msg and "wrong shape or dtype (1)" in msg


def test_optional_tensors_and_tied_head(tmp_path):
    d, cfg, _ = make_model_dir("tiny_qwen2", tmp_path)
    w = read_weights(d)
    assert "lm_head.weight" not in w and "model.layers.0.self_attn.q_proj.bias" in w
    w["lm_head.weight"] = torch.zeros(cfg["vocab_size"], cfg["hidden_size"])   # a tied model that stores one anyway
    write_file(os.path.join(d, "model.safetensors"), w)
    m = load_model(d, "float32", "cpu", ops=PlainOps())
    assert m.lm_head is m.embed
    d2, cfg2, _ = make_model_dir("tiny_llama", tmp_path)
    w2 = read_weights(d2)
    assert "lm_head.weight" in w2 and not any(k.endswith(".bias") for k in w2)
    m2 = load_model(d2, "float32", "cpu", ops=PlainOps())
    assert m2.lm_head is not m2.embed and m2.layers[0].mixer.bqkv is None
    del w2["lm_head.weight"]                                             # untied, none stored: the embedding is used
    write_file(os.path.join(d2, "model.safetensors"), w2)
    m3 = load_model(d2, "float32", "cpu", ops=PlainOps())
    assert m3.lm_head is m3.embed


def test_dtype_policy(tmp_path):
    d, cfg, _ = make_model_dir("tiny_qwen2", tmp_path, "float32")
    m = load_model(d, "bfloat16", "cpu", ops=PlainOps(torch.bfloat16))
    assert m.embed.dtype == torch.bfloat16 and m.layers[0].mixer.wqkv.dtype == torch.bfloat16
    assert m.final_norm.weight.dtype == torch.float32, "a 1-D tensor stored in 32-bit stays so"
    w = read_weights(d)
    assert torch.equal(m.embed, w["model.embed_tokens.weight"].to(torch.bfloat16))
    db, _, _ = make_model_dir("tiny_qwen2", tmp_path, "bfloat16")
    mb = load_model(db, "bfloat16", "cpu", ops=PlainOps(torch.bfloat16))
    assert mb.final_norm.weight.dtype == torch.bfloat16 and torch.equal(mb.embed, m.embed), "one seed, one model"
    mf = load_model(db, "float32", "cpu", ops=PlainOps())
    assert mf.embed.dtype == torch.float32 and mf.final_norm.weight.dtype == torch.float32


def test_random_weights_mode(tmp_path):
    cfg, o = get("tiny_llama")
    a = write_random_model(cfg, str(tmp_path / "a"), seed=3)
    b = write_random_model(cfg, str(tmp_path / "b"), seed=3)
    c = write_random_model(cfg, str(tmp_path / "c"), seed=4)
    wa, wb, wc = read_weights(a), read_weights(b), read_weights(c)
    assert all(torch.equal(wa[k], wb[k]) for k in wa) and not torch.equal(wa["lm_head.weight"], wc["lm_head.weight"])
    assert json.load(open(os.path.join(a, "config.json"))) == cfg
    assert set(wa) == {k for k, p in declared_tensors(describe(cfg)[1]).items() if p.group in (None, "lm_head")}
    assert torch.equal(wa["model.norm.weight"], torch.ones(64))
    emb = wa["model.embed_tokens.weight"]
    assert abs(float(emb.std()) - 0.02) < 0.002 and abs(float(emb.mean())) < 0.002
    noisy = read_weights(write_random_model(cfg, str(tmp_path / "n"), seed=3, norm_noise=True))
    assert 0.01 < float((noisy["model.norm.weight"] - 1).std()) < 0.03


def test_unknown_architecture_and_missing_files(tmp_path):
    os.makedirs(tmp_path / "m")
    with pytest.raises(FileNotFoundError, match="config.json"):
        load_model(str(tmp_path / "m"), "float32", "cpu", ops=PlainOps())
    with open(tmp_path / "m" / "config.json", "w") as f:
        json.dump({"model_type": "rwkv"}, f)
    with pytest.raises(NotImplementedError, match="rwkv"):
        load_model(str(tmp_path / "m"), "float32", "cpu", ops=PlainOps())
    with pytest.raises(ValueError, match="float16"):
        load_model(str(tmp_path / "m"), "float16", "cpu", ops=PlainOps())
