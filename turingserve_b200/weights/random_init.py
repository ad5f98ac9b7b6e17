"""Random-weights mode: write a model folder (config.json, model.safetensors) from a
configuration and a seed.

The reference makes tiny models through Hugging Face ``save_pretrained``
(scripts/make_tiny_model.py:22-42); here the folder is written directly: every tensor the model
declares, in declaration order, from one ``torch.Generator`` on the CPU: N(0, std) for
matrices, embeddings and biases, ones for norm scales.  The folder then loads like any checkpoint.
"""

from __future__ import annotations

import json
import os

import torch
from safetensors.torch import save_file

from turingserve_b200.config.model_config import ModelConfig
from turingserve_b200.config.registry import get_architecture
from turingserve_b200.parts.model import DecoderModel


def random_tensors(cfg: ModelConfig, seed: int, std: float = 0.02,
                   dtype: torch.dtype = torch.bfloat16) -> dict[str, torch.Tensor]:
    arch = get_architecture(cfg.architecture)
    names = arch.tensor_names(cfg)
    shell = DecoderModel(cfg, dtype, "cpu", max_positions=1)      # declares parameters; holds no weights
    g = torch.Generator(device="cpu").manual_seed(seed)
    out: dict[str, torch.Tensor] = {}
    for name, spec in shell.parameters(names).items():
        if spec.integer:
            out[name] = torch.zeros(spec.shape, dtype=torch.int32)
        elif spec.init == "ones":
            out[name] = torch.ones(spec.shape, dtype=dtype)
        elif spec.init == "zeros":
            out[name] = torch.zeros(spec.shape, dtype=dtype)
        else:
            out[name] = (torch.randn(spec.shape, generator=g, dtype=torch.float32) * std).to(dtype)
    return out


def write_random_model(folder: str, cfg: ModelConfig, seed: int, std: float = 0.02,
                       dtype: torch.dtype = torch.bfloat16) -> str:
    """Write ``folder/config.json`` and ``folder/model.safetensors``; returns ``folder``."""
    os.makedirs(folder, exist_ok=True)
    arch = get_architecture(cfg.architecture)
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as f:
        json.dump(arch.to_config_json(cfg), f, indent=1)
    save_file(random_tensors(cfg, seed, std, dtype), os.path.join(folder, "model.safetensors"))
    return folder
