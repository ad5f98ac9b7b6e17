"""Configuration: config.json keys -> ModelConfig, the registry, engine options, the command line."""

from __future__ import annotations

import json

import pytest

from turingserve_b200.config import EngineConfig, load_model_config
from turingserve_b200.config.engine_config import add_engine_arguments, engine_config_from_namespace
from turingserve_b200.config.registry import architecture_of, get_architecture
from turingserve_b200.models import qwen2

BASE = {"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "hidden_size": 96, "intermediate_size": 224,
        "num_hidden_layers": 3, "num_attention_heads": 3, "num_key_value_heads": 1, "vocab_size": 320,
        "rope_theta": 1e6, "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "max_position_embeddings": 256}


def test_every_size_comes_from_config_json():
    c = qwen2.parse_config(BASE)
    a = c.layers[0].mixer
    assert (c.hidden_size, c.vocab_size, len(c.layers)) == (96, 320, 3)
    assert (a.num_heads, a.num_kv_heads, a.head_dim) == (3, 1, 32)
    assert a.scale == 32 ** -0.5 and a.qkv_bias and not a.out_bias and a.window is None
    assert a.position.theta == 1e6 and a.position.rotary_dim == 32 and a.position.max_positions == 256
    assert c.layers[0].feed_forward.intermediate_size == 224
    assert c.final_norm.eps == 1e-5 and c.layers[2].mixer_norm.eps == 1e-5
    assert not c.tie_word_embeddings and c.eos_token_ids == ()
    assert [r.layer for r in c.schedule] == [0, 1, 2] and all(r.cache_from is None for r in c.schedule)


def test_optional_keys_and_defaults():
    c = qwen2.parse_config({**BASE, "head_dim": 48, "eos_token_id": [7, 9], "bos_token_id": 1})
    assert c.layers[0].mixer.head_dim == 48 and c.eos_token_ids == (7, 9) and c.bos_token_id == 1
    d = dict(BASE)
    del d["rope_theta"], d["rms_norm_eps"]
    c = qwen2.parse_config({**d, "rope_parameters": {"rope_theta": 5e5}})
    assert c.layers[0].mixer.position.theta == 5e5 and c.final_norm.eps == 1e-6
    assert qwen2.parse_config(d).layers[0].mixer.position.theta == 10000.0
    c = qwen2.parse_config(BASE, {"eos_token_id": 5})          # generation_config.json wins
    assert c.eos_token_ids == (5,)


def test_window_layers():
    c = qwen2.parse_config({**BASE, "use_sliding_window": True, "sliding_window": 24, "max_window_layers": 1})
    assert [l.mixer.window for l in c.layers] == [None, 24, 24]
    c = qwen2.parse_config({**BASE, "use_sliding_window": False, "sliding_window": 24})
    assert [l.mixer.window for l in c.layers] == [None] * 3


@pytest.mark.parametrize("patch,msg", [
    ({"model_type": "llama"}, "model_type"), ({"rope_scaling": {"type": "yarn"}}, "rope_scaling"),
    ({"num_key_value_heads": 2}, "multiple"), ({"hidden_act": "gelu"}, "hidden_act"),
    ({"rope_parameters": {"rope_type": "linear"}}, "rope_type")])
def test_rejects(patch, msg):
    with pytest.raises(ValueError, match=msg):
        qwen2.parse_config({**BASE, **patch})


def test_missing_key_is_named():
    d = dict(BASE)
    del d["intermediate_size"]
    with pytest.raises(ValueError, match="intermediate_size"):
        qwen2.parse_config(d)


def test_registry(tmp_path):
    assert architecture_of(BASE).name == "Qwen2ForCausalLM"
    with pytest.raises(ValueError, match="unknown architecture"):
        get_architecture("NoSuchModel")
    with pytest.raises(ValueError, match="architectures"):
        architecture_of({"model_type": "qwen2"})
    (tmp_path / "config.json").write_text(json.dumps(BASE))
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": [3, 4]}))
    assert load_model_config(str(tmp_path)).eos_token_ids == (3, 4)
    with pytest.raises(FileNotFoundError):
        load_model_config(str(tmp_path / "nothing"))


def test_config_json_round_trip():
    c = qwen2.parse_config({**BASE, "use_sliding_window": True, "sliding_window": 24, "max_window_layers": 1,
                            "head_dim": 48, "eos_token_id": 2})
    assert qwen2.parse_config(qwen2.to_config_json(c)) == c


def test_schedule_validation():
    from turingserve_b200.config import LayerRun
    c = qwen2.parse_config(BASE)
    c.with_schedule([LayerRun(0), LayerRun(1), LayerRun(1, cache_from=1), LayerRun(0)])
    with pytest.raises(ValueError, match="earlier"):
        c.with_schedule([LayerRun(0, cache_from=0)])
    with pytest.raises(ValueError, match="names layer"):
        c.with_schedule([LayerRun(5)])
    with pytest.raises(ValueError, match="without a cache"):
        c.with_schedule([LayerRun(0), LayerRun(1, cache_from=0), LayerRun(2, cache_from=1)])


def test_engine_config_validation_and_cli():
    import argparse
    p = argparse.ArgumentParser()
    add_engine_arguments(p)
    ns = p.parse_args(["--model", "m", "--dtype", "float32", "--max-model-len", "512", "--block-size", "8",
                       "--num-blocks", "40", "--max-num-seqs", "4", "--max-num-batched-tokens", "64",
                       "--watermark", "0.05", "--no-cuda-graphs", "--graph-batch-sizes", "1,2,8", "--seed", "3"])
    cfg = engine_config_from_namespace(ns)
    assert (cfg.model, cfg.dtype, cfg.max_model_len, cfg.block_size, cfg.num_blocks) == ("m", "float32", 512, 8, 40)
    assert (cfg.max_num_seqs, cfg.max_num_batched_tokens, cfg.watermark, cfg.cuda_graphs) == (4, 64, 0.05, False)
    assert cfg.graph_batch_sizes == (1, 2, 8) and cfg.seed == 3
    cfg.validate(1024)
    assert cfg.graph_batch_sizes == (1, 2)                        # sizes above max_num_seqs are dropped
    assert cfg.max_blocks_per_seq(512) == 64
    with pytest.raises(ValueError, match="exceeds"):
        cfg.validate(256)
    for bad in (dict(model=""), dict(dtype="float16"), dict(device="cpu"), dict(num_blocks=1),
                dict(watermark=1.5), dict(max_num_seqs=0), dict(gpu_memory_utilization=0.0)):
        with pytest.raises(ValueError):
            EngineConfig(**{"model": "m", **bad}).validate()
    assert EngineConfig(model="m").resolve_max_model_len(32768) == 4096
    assert EngineConfig(model="m").resolve_max_model_len(128) == 128


def test_a_head_size_no_attention_kernel_takes_is_refused_when_the_model_is_built():
    import torch

    from turingserve_b200.parts.model import DecoderModel
    cfg = qwen2.parse_config({**BASE, "hidden_size": 96, "num_attention_heads": 3, "head_dim": 272})
    with pytest.raises(ValueError, match="head sizes up to 256"):
        DecoderModel(cfg, torch.float32, "cpu", 16)
    DecoderModel(qwen2.parse_config({**BASE, "head_dim": 256}), torch.float32, "cpu", 16)


def test_captured_portion_lengths_follow_the_token_budget():
    """Token budgets up to `graph_portion_budget` capture steps of decoding requests beside one prompt
    portion: the portion lengths are the budget less each captured batch size (and less none), down to 16
    tokens; larger budgets, or no graphs, capture none."""
    from turingserve_b200 import EngineConfig
    c = EngineConfig(model="m", max_num_batched_tokens=512, graph_batch_sizes=(1, 2, 4, 8, 16, 32, 64, 128))
    assert c.graph_portion_sizes() == (384, 448, 480, 496, 504, 508, 510, 511, 512)
    assert EngineConfig(model="m", max_num_batched_tokens=40, graph_batch_sizes=(1, 8, 32)).graph_portion_sizes() == (32, 39, 40)
    assert EngineConfig(model="m", max_num_batched_tokens=2048).graph_portion_sizes() == ()
    assert EngineConfig(model="m", max_num_batched_tokens=2048, graph_portion_budget=4096).graph_portion_sizes()[-1] == 2048
    assert EngineConfig(model="m", max_num_batched_tokens=512, cuda_graphs=False).graph_portion_sizes() == ()
    assert EngineConfig(model="m", max_num_batched_tokens=512, graph_portion_budget=0).graph_portion_sizes() == ()
