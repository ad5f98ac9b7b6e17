"""Weights from safetensors, bound by tensor name.

File discovery and "every tensor is used" follow turingserve/model/loader.py:19-52,94-98; unlike
the reference (which raises at the first missing name, loader.py:41-43) all problems are collected
and reported in ONE error: missing tensors, unexpected tensors, wrong shapes.

Precision: floating tensors that feed matrix products are kept in the engine's dtype (bfloat16
or float32); a tensor a part marks ``compute_dtype=False`` stays in 32-bit if it is stored so;
integer tables become int32.
"""

from __future__ import annotations

import glob
import json
import os

import torch
from safetensors import safe_open

from turingserve_b200.config.model_config import ModelConfig
from turingserve_b200.config.registry import architecture_of, read_config_json
from turingserve_b200.parts.base import ParamSpec
from turingserve_b200.parts.model import DecoderModel


class WeightsError(ValueError):
    """The checkpoint does not fit the model; the message lists every mismatch."""

    def __init__(self, missing, unexpected, wrong_shape, where: str) -> None:
        self.missing, self.unexpected, self.wrong_shape = list(missing), list(unexpected), list(wrong_shape)
        lines = [f"checkpoint {where!r} does not fit the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}): " + ", ".join(
                f"{n} is {list(got)}, expected {list(exp)}" for n, got, exp in self.wrong_shape))
        super().__init__("\n".join(lines))


def tensor_files(path: str) -> dict[str, str]:
    """Tensor name -> file, from ``model.safetensors.index.json`` or all ``*.safetensors``."""
    index = os.path.join(path, "model.safetensors.index.json")
    if os.path.exists(index):
        with open(index, encoding="utf-8") as f:
            wm = json.load(f)["weight_map"]
        return {k: os.path.join(path, v) for k, v in wm.items()}
    out: dict[str, str] = {}
    for fn in sorted(glob.glob(os.path.join(path, "*.safetensors"))):
        with safe_open(fn, framework="pt", device="cpu") as f:
            for k in f.keys():
                out[k] = fn
    if not out:
        raise FileNotFoundError(f"no *.safetensors files in {path!r}")
    return out


def _convert(t: torch.Tensor, spec: ParamSpec, dtype: torch.dtype, name: str) -> torch.Tensor:
    if spec.integer:
        if t.dtype.is_floating_point:
            raise ValueError(f"{name}: expected an integer table, file has {t.dtype}")
        return t.to(torch.int32)
    if not t.dtype.is_floating_point:
        raise ValueError(f"{name}: expected a floating tensor, file has {t.dtype}")
    if not spec.compute_dtype and t.dtype == torch.float32:
        out = t
    else:
        out = t.to(dtype)
    if not torch.isfinite(out).all():
        raise ValueError(f"non-finite values in {name} after conversion to {out.dtype}")
    return out


def load_into(model: DecoderModel, model_dir: str, names=None) -> None:
    """Read every tensor ``model`` declares from ``model_dir`` and hand them over."""
    arch_names = names
    if arch_names is None:
        from turingserve_b200.config.registry import get_architecture
        arch_names = get_architecture(model.cfg.architecture).tensor_names(model.cfg)
    expected = model.parameters(arch_names)
    files = tensor_files(model_dir)

    handles: dict[str, object] = {}

    def handle(fn: str):
        if fn not in handles:
            handles[fn] = safe_open(fn, framework="pt", device="cpu")
        return handles[fn]

    missing = [n for n in expected if n not in files]
    unexpected = sorted(n for n in files if n not in expected and n not in arch_names.tolerated)
    wrong = []
    for n, spec in expected.items():
        if n in files:
            got = tuple(handle(files[n]).get_slice(n).get_shape())
            if got != tuple(spec.shape):
                wrong.append((n, got, tuple(spec.shape)))
    if missing or unexpected or wrong:
        raise WeightsError(missing, unexpected, wrong, model_dir)

    tensors: dict[str, torch.Tensor] = {}
    for n, spec in expected.items():
        t = handle(files[n]).get_tensor(n)
        tensors[n] = _convert(t, spec, model.dtype, n).to(model.device)
    model.load(arch_names, tensors)


def load_model(model_dir: str, dtype: torch.dtype, device, max_positions: int | None = None
               ) -> tuple[DecoderModel, ModelConfig]:
    """``config.json`` chooses the architecture; returns the model with weights on ``device``."""
    cfg_json, gen = read_config_json(model_dir)
    arch = architecture_of(cfg_json)
    cfg = arch.parse_config(cfg_json, gen)
    model = (arch.build_model or DecoderModel)(cfg, dtype, device, max_positions or cfg.max_position_embeddings)
    load_into(model, model_dir, arch.tensor_names(cfg))
    return model, cfg
