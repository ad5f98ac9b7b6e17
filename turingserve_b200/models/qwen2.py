"""Qwen2 / Qwen2.5 dense decoder: config.json keys -> ``ModelConfig``, and checkpoint tensor names.

The recipe (what is fixed for this family, as opposed to read from config.json):
pre-norm blocks; RMSNorm; grouped-query attention with bias on q/k/v and none on the output
projection; rotate-half rotary encoding over the whole head; gated SiLU feed-forward without
bias; score scale head_dim**-0.5.  Sources: turingserve/model/qwen2.py:19,24-61,
turingserve/model/qwen2_config.py:36-63, turingserve/model/loader.py:78-93.

Beyond the reference: ``head_dim`` is honoured when config.json has it, untied ``lm_head`` is
supported, and ``use_sliding_window`` builds windowed attention layers (the reference rejects it,
qwen2_config.py:40-41): by the meaning of the config keys, the first ``max_window_layers`` layers
attend to everything and the layers after them to the last ``sliding_window`` positions.
"""

from __future__ import annotations

from turingserve_b200.config.model_config import (
    AttentionSpec, GatedMLPSpec, LayerRun, LayerSpec, ModelConfig, RMSNormSpec, RotarySpec)
from turingserve_b200.config.registry import (
    Architecture, LayerTensorNames, TensorNames, register_architecture)

NAME = "Qwen2ForCausalLM"


def _require(c: dict, key: str):
    if key not in c:
        raise ValueError(f"config.json is missing required key {key!r}")
    return c[key]


def parse_config(c: dict, gen: dict | None = None) -> ModelConfig:
    if c.get("model_type", "qwen2") != "qwen2":
        raise ValueError(f"unsupported model_type {c.get('model_type')!r} for {NAME}")
    if c.get("rope_scaling"):
        raise ValueError("rope_scaling is not supported")
    rp = c.get("rope_parameters") or {}
    if rp.get("rope_type", "default") != "default":
        raise ValueError(f"rope_type {rp['rope_type']!r} is not supported")
    theta = float(c.get("rope_theta", rp.get("rope_theta", 10000.0)))
    hidden = int(_require(c, "hidden_size"))
    heads = int(_require(c, "num_attention_heads"))
    kv_heads = int(_require(c, "num_key_value_heads"))
    if heads % kv_heads:
        raise ValueError("num_attention_heads must be a multiple of num_key_value_heads")
    head_dim = int(c["head_dim"]) if c.get("head_dim") else hidden // heads
    if head_dim % 2:
        raise ValueError("head_dim must be even for rotate-half rotary encoding")
    act = c.get("hidden_act", "silu")
    if act != "silu":
        raise ValueError(f"hidden_act {act!r} is not supported")
    n_layers = int(_require(c, "num_hidden_layers"))
    max_pos = int(_require(c, "max_position_embeddings"))
    eps = float(c.get("rms_norm_eps", 1e-6))

    window = None
    first_window_layer = n_layers
    if c.get("use_sliding_window"):
        window = int(_require(c, "sliding_window"))
        if window < 1:
            raise ValueError("sliding_window must be >= 1")
        first_window_layer = int(c.get("max_window_layers", n_layers))

    eos = (gen or {}).get("eos_token_id", c.get("eos_token_id"))
    if eos is None:
        eos = ()
    eos_ids = (int(eos),) if isinstance(eos, int) else tuple(int(x) for x in eos)

    rotary = RotarySpec(theta=theta, rotary_dim=head_dim, max_positions=max_pos)
    norm = RMSNormSpec(eps=eps)
    ffn = GatedMLPSpec(intermediate_size=int(_require(c, "intermediate_size")), activation=act, bias=False)
    layers = []
    for i in range(n_layers):
        mixer = AttentionSpec(
            num_heads=heads, num_kv_heads=kv_heads, head_dim=head_dim, scale=head_dim ** -0.5,
            qkv_bias=True, out_bias=False, position=rotary,
            window=window if i >= first_window_layer else None)
        layers.append(LayerSpec(mixer=mixer, feed_forward=ffn, mixer_norm=norm, ffn_norm=norm))
    return ModelConfig(
        architecture=NAME, hidden_size=hidden, vocab_size=int(_require(c, "vocab_size")),
        layers=tuple(layers), schedule=tuple(LayerRun(i) for i in range(n_layers)),
        final_norm=norm, tie_word_embeddings=bool(c.get("tie_word_embeddings", False)),
        max_position_embeddings=max_pos, eos_token_ids=eos_ids, bos_token_id=c.get("bos_token_id"))


def tensor_names(cfg: ModelConfig) -> TensorNames:
    """HF tensor names (turingserve/model/loader.py:78-93)."""
    layers = tuple(
        LayerTensorNames(
            mixer=f"model.layers.{i}.self_attn.", feed_forward=f"model.layers.{i}.mlp.",
            mixer_norm=f"model.layers.{i}.input_layernorm.",
            ffn_norm=f"model.layers.{i}.post_attention_layernorm.")
        for i in range(len(cfg.layers)))
    return TensorNames(
        embedding="model.embed_tokens.weight", lm_head="lm_head.weight", final_norm="model.norm.",
        layers=layers, tolerated=("lm_head.weight",) if cfg.tie_word_embeddings else ())


def to_config_json(cfg: ModelConfig) -> dict:
    a = cfg.layers[0].mixer
    windows = [l.mixer.window for l in cfg.layers]
    first_w = next((i for i, w in enumerate(windows) if w is not None), len(windows))
    out = {
        "architectures": [NAME], "model_type": "qwen2",
        "hidden_size": cfg.hidden_size, "intermediate_size": cfg.layers[0].feed_forward.intermediate_size,
        "num_hidden_layers": len(cfg.layers), "num_attention_heads": a.num_heads,
        "num_key_value_heads": a.num_kv_heads, "head_dim": a.head_dim, "vocab_size": cfg.vocab_size,
        "rms_norm_eps": cfg.final_norm.eps, "rope_theta": a.position.theta,
        "max_position_embeddings": cfg.max_position_embeddings, "hidden_act": "silu",
        "tie_word_embeddings": cfg.tie_word_embeddings,
        "use_sliding_window": first_w < len(windows),
    }
    if first_w < len(windows):
        out["sliding_window"] = windows[first_w]
        out["max_window_layers"] = first_w
    if cfg.eos_token_ids:
        out["eos_token_id"] = list(cfg.eos_token_ids) if len(cfg.eos_token_ids) > 1 else cfg.eos_token_ids[0]
    if cfg.bos_token_id is not None:
        out["bos_token_id"] = cfg.bos_token_id
    return out


def make_config(*, hidden_size: int, intermediate_size: int, num_layers: int, num_heads: int,
                num_kv_heads: int, vocab_size: int, head_dim: int | None = None,
                rope_theta: float = 10000.0, rms_norm_eps: float = 1e-6,
                tie_word_embeddings: bool = False, max_position_embeddings: int = 4096,
                sliding_window: int | None = None, max_window_layers: int | None = None,
                eos_token_id: int | None = None) -> ModelConfig:
    """Build a Qwen2 ``ModelConfig`` from sizes (goes through the same parser as config.json)."""
    c = {
        "architectures": [NAME], "model_type": "qwen2", "hidden_size": hidden_size,
        "intermediate_size": intermediate_size, "num_hidden_layers": num_layers,
        "num_attention_heads": num_heads, "num_key_value_heads": num_kv_heads,
        "vocab_size": vocab_size, "rope_theta": rope_theta, "rms_norm_eps": rms_norm_eps,
        "tie_word_embeddings": tie_word_embeddings, "max_position_embeddings": max_position_embeddings,
    }
    if head_dim is not None:
        c["head_dim"] = head_dim
    if sliding_window is not None:
        c.update(use_sliding_window=True, sliding_window=sliding_window,
                 max_window_layers=num_layers if max_window_layers is None else max_window_layers)
    if eos_token_id is not None:
        c["eos_token_id"] = eos_token_id
    return parse_config(c)


register_architecture(Architecture(NAME, parse_config, tensor_names, to_config_json))
