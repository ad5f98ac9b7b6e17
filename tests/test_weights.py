"""Weights: the random-weights writer, loading by name, and the one error that lists everything."""

from __future__ import annotations

import os

import pytest
import torch
from safetensors.torch import load_file, save_file

from tests import tiny
from turingserve_b200.weights import WeightsError, load_model, random_tensors, write_random_model


def test_random_model_folder_is_deterministic_and_loads(tmp_path):
    f1 = tiny.make_tiny_folder("B", tmp_path / "a")
    f2 = tiny.make_tiny_folder("B", tmp_path / "b")
    t1, t2 = load_file(os.path.join(f1, "model.safetensors")), load_file(os.path.join(f2, "model.safetensors"))
    assert t1.keys() == t2.keys() and all(torch.equal(t1[k], t2[k]) for k in t1)
    assert "lm_head.weight" in t1 and t1["model.layers.2.self_attn.k_proj.bias"].shape == (32,)
    assert all(v.dtype == torch.bfloat16 for v in t1.values())
    assert torch.all(t1["model.norm.weight"] == 1)
    other = random_tensors(tiny.tiny_config("B"), seed=2)
    assert not torch.equal(other["model.embed_tokens.weight"], t1["model.embed_tokens.weight"])
    for dtype in (torch.float32, torch.bfloat16):
        model, cfg = load_model(f1, dtype, "cpu")
        att = model.blocks[0].mixer
        assert att.w_qkv.shape == (5 * 32, 96) and att.w_qkv.dtype == dtype
        q = t1["model.layers.0.self_attn.q_proj.weight"].to(dtype)
        assert torch.equal(att.w_qkv[:96], q)                   # fused in the order q, k, v
        assert model.blocks[1].feed_forward.w_gate_up.shape == (448, 96)
        assert model.lm_head is not model.embedding and model.embedding.dtype == dtype


def test_tied_head_shares_the_embedding(tmp_path):
    f = tiny.make_tiny_folder("A", tmp_path)
    model, cfg = load_model(f, torch.float32, "cpu")
    assert model.lm_head is model.embedding
    assert "lm_head.weight" not in load_file(os.path.join(f, "model.safetensors"))


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    f = tiny.make_tiny_folder("A", tmp_path)
    path = os.path.join(f, "model.safetensors")
    t = load_file(path)
    del t["model.layers.1.mlp.up_proj.weight"]
    del t["model.norm.weight"]
    t["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    t["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(7, dtype=torch.bfloat16)
    t["model.embed_tokens.weight"] = torch.zeros(256, 32, dtype=torch.bfloat16)
    save_file(t, path)
    with pytest.raises(WeightsError) as e:
        load_model(f, torch.float32, "cpu")
    err = e.value
    assert sorted(err.missing) == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.0.self_attn.rotary_emb.inv_freq"]
    assert sorted(n for n, _, _ in err.wrong_shape) == ["model.embed_tokens.weight", "model.layers.0.self_attn.q_proj.bias"]
    msg = str(err)
    for piece in ("missing tensors (2)", "unexpected tensors (1)", "wrong shapes (2)", "is [7], expected [64]"):
        assert piece in msg


def test_tied_checkpoint_may_carry_a_duplicate_head_but_untied_needs_it(tmp_path):
    f = tiny.make_tiny_folder("A", tmp_path)
    path = os.path.join(f, "model.safetensors")
    t = load_file(path)
    t["lm_head.weight"] = t["model.embed_tokens.weight"].clone()
    save_file(t, path)
    load_model(f, torch.float32, "cpu")
    fb = tiny.make_tiny_folder("B", tmp_path)
    tb = load_file(os.path.join(fb, "model.safetensors"))
    del tb["lm_head.weight"]
    save_file(tb, os.path.join(fb, "model.safetensors"))
    with pytest.raises(WeightsError, match="lm_head.weight"):
        load_model(fb, torch.float32, "cpu")


def test_precision_rules(tmp_path):
    """bfloat16 stays bfloat16; a scale stored in 32-bit stays 32-bit; matrices follow the engine's dtype."""
    f = tiny.make_tiny_folder("A", tmp_path)
    path = os.path.join(f, "model.safetensors")
    t = load_file(path)
    t["model.norm.weight"] = t["model.norm.weight"].float() * 1.0009765625       # not a bfloat16 number
    t["model.layers.0.mlp.down_proj.weight"] = t["model.layers.0.mlp.down_proj.weight"].float()
    save_file(t, path)
    model, _ = load_model(f, torch.bfloat16, "cpu")
    assert model.final_norm.weight.dtype == torch.float32
    assert model.final_norm.weight[0].item() == pytest.approx(1.0009765625)
    assert model.blocks[0].feed_forward.w_down.dtype == torch.bfloat16
    assert model.blocks[0].mixer_norm.weight.dtype == torch.bfloat16
    t["model.layers.1.self_attn.o_proj.weight"][0, 0] = float("nan")
    save_file(t, path)
    with pytest.raises(ValueError, match="non-finite"):
        load_model(f, torch.bfloat16, "cpu")


def test_sharded_checkpoint_with_index(tmp_path):
    import json
    f = tiny.make_tiny_folder("A", tmp_path)
    t = load_file(os.path.join(f, "model.safetensors"))
    os.remove(os.path.join(f, "model.safetensors"))
    names = sorted(t)
    a, b = names[: len(names) // 2], names[len(names) // 2:]
    save_file({k: t[k] for k in a}, os.path.join(f, "model-00001-of-00002.safetensors"))
    save_file({k: t[k] for k in b}, os.path.join(f, "model-00002-of-00002.safetensors"))
    wm = {k: "model-00001-of-00002.safetensors" for k in a} | {k: "model-00002-of-00002.safetensors" for k in b}
    with open(os.path.join(f, "model.safetensors.index.json"), "w") as fh:
        json.dump({"weight_map": wm}, fh)
    load_model(f, torch.float32, "cpu")
    os.remove(os.path.join(f, "model.safetensors.index.json"))
    load_model(f, torch.float32, "cpu")                           # glob of *.safetensors
    with pytest.raises(FileNotFoundError):
        load_model(str(tmp_path), torch.float32, "cpu") if False else load_model(_empty(tmp_path, f), torch.float32, "cpu")


def _empty(tmp_path, f):
    import shutil
    d = tmp_path / "empty"
    d.mkdir()
    shutil.copy(os.path.join(f, "config.json"), d / "config.json")
    return str(d)
