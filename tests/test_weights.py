"""Weights: the container, the random-weights mode, and the loader's one error."""
import json
import os

import pytest
import torch

from crucible_b200.config import parse_config
from crucible_b200.models.decoder import DecoderModel
from crucible_b200.weights import (SafetensorsFile, WeightError, load_weights,
                                   write_random_model, write_safetensors)
from helpers import TINY


def test_container_round_trip(tmp_path):
    tensors = {"a": torch.randn(3, 5), "b": torch.randn(7).bfloat16(),
               "c": torch.arange(6, dtype=torch.int32).view(2, 3), "empty": torch.zeros(0, 4)}
    path = str(tmp_path / "x.safetensors")
    write_safetensors(path, tensors, {"format": "pt"})
    f = SafetensorsFile(path)
    assert sorted(f.names()) == sorted(tensors)
    for k, v in tensors.items():
        got = f.get(k)
        assert got.dtype == v.dtype and torch.equal(got, v)
    f.close()
    # the other implementation of the format reads it too
    from safetensors import safe_open
    with safe_open(path, framework="pt") as g:
        assert torch.equal(g.get_tensor("b"), tensors["b"])


def test_random_model_folder_is_deterministic(tmp_path):
    a = write_random_model(TINY["tiny-a"]["config"], str(tmp_path / "a"), seed=5)
    b = write_random_model(TINY["tiny-a"]["config"], str(tmp_path / "b"), seed=5)
    c = write_random_model(TINY["tiny-a"]["config"], str(tmp_path / "c"), seed=6)
    fa, fb, fc = (SafetensorsFile(os.path.join(d, "model.safetensors")) for d in (a, b, c))
    assert fa.names() == fb.names()
    for n in fa.names():
        assert torch.equal(fa.get(n), fb.get(n))
    assert not torch.equal(fa.get("tok_emb.weight"), fc.get("tok_emb.weight"))
    assert "lm_head.weight" not in fa                       # tied: stored once
    assert fa.get("tok_emb.weight").dtype == torch.bfloat16
    assert fa.get("final_norm.weight").dtype == torch.float32
    assert torch.all(fa.get("blocks.1.attn_norm.weight") == 1)
    std = float(fa.get("blocks.0.mlp.up_proj.weight").float().std())
    assert 0.015 < std < 0.025
    cfg = json.load(open(os.path.join(a, "config.json")))
    assert parse_config(cfg) == parse_config(TINY["tiny-a"]["config"])
    b_dir = write_random_model(TINY["tiny-b"]["config"], str(tmp_path / "tb"), seed=2,
                               store_dtype="float32")
    fb2 = SafetensorsFile(os.path.join(b_dir, "model.safetensors"))
    assert fb2.get("lm_head.weight").dtype == torch.float32   # untied: its own matrix


def _model(name):
    return DecoderModel(parse_config(TINY[name]["config"]))


def test_loader_keeps_dtypes_by_role(tmp_path):
    folder = write_random_model(TINY["tiny-a"]["config"], str(tmp_path / "m"), seed=1)
    m = _model("tiny-a")
    load_weights(m, folder, torch.bfloat16, "cpu")
    assert m.embedding.table.dtype == torch.bfloat16
    assert m.final_norm.gain.dtype == torch.float32          # a vector stays in 32 bits
    assert m.head.weight is m.embedding.table                # tied
    assert m.layers[0].mixer.wqkv.shape == ((4 + 2 * 2) * 16, 64)
    m32 = _model("tiny-a")
    load_weights(m32, folder, torch.float32, "cpu")
    assert m32.layers[1].feed_forward.gate_up.dtype == torch.float32
    assert torch.equal(m32.embedding.table, m.embedding.table.float())   # widened exactly


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    folder = write_random_model(TINY["tiny-a"]["config"], str(tmp_path / "m"), seed=1)
    path = os.path.join(folder, "model.safetensors")
    f = SafetensorsFile(path)
    tensors = {n: f.get(n) for n in f.names()}
    f.close()
    del tensors["blocks.0.attn.k_proj.weight"]
    del tensors["final_norm.weight"]
    tensors["blocks.0.attn.rotary.inv_freq"] = torch.zeros(8)
    tensors["blocks.1.mlp.down_proj.weight"] = torch.zeros(64, 175).bfloat16()
    tensors["blocks.1.mlp_norm.weight"] = torch.zeros(64, dtype=torch.int32)
    write_safetensors(path, tensors)
    with pytest.raises(WeightError) as e:
        load_weights(_model("tiny-a"), folder, torch.float32, "cpu")
    err = e.value
    assert err.missing == ["final_norm.weight", "blocks.0.attn.k_proj.weight"] or \
        sorted(err.missing) == ["blocks.0.attn.k_proj.weight", "final_norm.weight"]
    assert err.unexpected == ["blocks.0.attn.rotary.inv_freq"]
    assert [w[0] for w in err.wrong_shape] == ["blocks.1.mlp.down_proj.weight"]
    assert [w[0] for w in err.wrong_dtype] == ["blocks.1.mlp_norm.weight"]
    text = str(err)
    for needle in ("missing tensors", "unexpected tensors", "[64, 175]", "[64, 176]",
                   "blocks.0.attn.k_proj.weight", "rotary.inv_freq"):
        assert needle in text


def test_missing_file_and_untied_head(tmp_path):
    os.makedirs(tmp_path / "empty")
    with pytest.raises(WeightError, match="no such weights file"):
        load_weights(_model("tiny-a"), str(tmp_path / "empty"), torch.float32, "cpu")
    folder = write_random_model(TINY["tiny-b"]["config"], str(tmp_path / "b"), seed=2)
    path = os.path.join(folder, "model.safetensors")
    f = SafetensorsFile(path)
    tensors = {n: f.get(n) for n in f.names() if n != "lm_head.weight"}
    f.close()
    write_safetensors(path, tensors)
    with pytest.raises(WeightError, match="lm_head.weight"):
        load_weights(_model("tiny-b"), folder, torch.bfloat16, "cpu")


def test_engine_dtype_is_checked(tmp_path):
    folder = write_random_model(TINY["tiny-a"]["config"], str(tmp_path / "m"), seed=1)
    with pytest.raises(ValueError):
        load_weights(_model("tiny-a"), folder, torch.float16, "cpu")
