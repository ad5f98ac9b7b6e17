"""Random-weights mode: write a model folder (config.json, model.safetensors) from a
configuration and a seed.

The reference makes tiny models through Hugging Face ``save_pretrained``
(scripts/make_tiny_model.py:22-42); here the folder is written directly: every tensor the model
declares, in declaration order, from one ``torch.Generator`` on the CPU: N(0, std) for
matrices, embeddings and biases, ones for norm scales.  The folder then loads like any checkpoint.

``random_model_on_device`` is the same recipe without the folder: the tensors are drawn on the
device and handed to the model directly, for measurements at sizes whose checkpoint would be
tens of gigabytes on disk.
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
    shell = (arch.build_model or DecoderModel)(cfg, dtype, "cpu", 1)      # declares parameters; holds no weights
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


def random_model_on_device(cfg: ModelConfig, dtype: torch.dtype, device, seed: int, std: float = 0.02,
                           max_positions: int | None = None) -> DecoderModel:
    """A model of configuration ``cfg`` with N(0, std) weights drawn on ``device`` (ones for norm
    scales): what ``write_random_model`` + ``load_model`` give, without the file in between and
    with the device's generator instead of the CPU's."""
    arch = get_architecture(cfg.architecture)
    names = arch.tensor_names(cfg)
    build = arch.build_model or DecoderModel
    model = build(cfg, dtype, device, max_positions or cfg.max_position_embeddings)
    g = torch.Generator(device=device).manual_seed(seed)
    tensors: dict[str, torch.Tensor] = {}
    for name, spec in model.parameters(names).items():
        kind = dtype if spec.compute_dtype else torch.float32
        if spec.integer:
            tensors[name] = torch.zeros(spec.shape, dtype=torch.int32, device=device)
        elif spec.init == "ones":
            tensors[name] = torch.ones(spec.shape, dtype=kind, device=device)
        elif spec.init == "zeros":
            tensors[name] = torch.zeros(spec.shape, dtype=kind, device=device)
        else:
            t = torch.empty(spec.shape, dtype=kind, device=device)
            t.normal_(0.0, std, generator=g)
            tensors[name] = t
    model.load(names, tensors)
    return model
