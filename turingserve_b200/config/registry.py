"""One registry from an architecture's name (``config.json`` -> ``architectures[0]``) to the
recipe that turns its configuration keys into a ``ModelConfig`` and names its checkpoint tensors.

The reference has no registry: ``build_engine`` imports Qwen2 directly and only checks
``model_type`` (turingserve/engine/builder.py:14-15,31,46; turingserve/model/qwen2_config.py:38-39).
"""

from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Callable

from turingserve_b200.config.model_config import ModelConfig


class LayerTensorNames:
    """Checkpoint prefix of every part of one layer, by the part's role in the layer (the role
    names of its ``LayerSpec``); each prefix ends with '.' or is ''.  ``names["mixer"]`` or
    ``names.mixer``."""

    def __init__(self, **prefixes: str) -> None:
        self._prefixes = dict(prefixes)

    def __getitem__(self, role: str) -> str:
        try:
            return self._prefixes[role]
        except KeyError:
            raise KeyError(f"the architecture names no checkpoint prefix for the layer part {role!r} "
                           f"(named: {', '.join(self._prefixes)})") from None

    def __getattr__(self, role: str) -> str:
        if role.startswith("_"):
            raise AttributeError(role)
        try:
            return self._prefixes[role]
        except KeyError:
            raise AttributeError(role) from None

    def roles(self) -> tuple[str, ...]:
        return tuple(self._prefixes)

    def __repr__(self) -> str:
        return f"LayerTensorNames({self._prefixes!r})"


@dataclass(frozen=True)
class TensorNames:
    """Where each part of a model finds its tensors in the checkpoint."""

    embedding: str
    lm_head: str
    final_norm: str
    layers: tuple[LayerTensorNames, ...]
    # names that may be present but are not read (e.g. a duplicate head in a tied checkpoint)
    tolerated: tuple[str, ...] = field(default_factory=tuple)


@dataclass(frozen=True)
class Architecture:
    name: str
    parse_config: Callable[[dict, dict | None], ModelConfig]
    tensor_names: Callable[[ModelConfig], TensorNames]
    # inverse of parse_config, used by the random-weights writer
    to_config_json: Callable[[ModelConfig], dict]
    # the model class: called as build_model(cfg, dtype, device, max_positions); None = the plain
    # decoder (turingserve_b200.parts.model.DecoderModel).  A family that scales its embeddings or
    # caps its logits registers a subclass that overrides ``embed`` / ``finish_logits``.
    build_model: Callable | None = None


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(arch: Architecture) -> None:
    _ARCHITECTURES[arch.name] = arch


def get_architecture(name: str) -> Architecture:
    _load_builtin()
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        known = ", ".join(sorted(_ARCHITECTURES)) or "none"
        raise ValueError(f"unknown architecture {name!r} (registered: {known})") from None


def architecture_of(config_json: dict) -> Architecture:
    archs = config_json.get("architectures")
    if not archs or not isinstance(archs, (list, tuple)):
        raise ValueError("config.json has no 'architectures' list; cannot choose a model class")
    return get_architecture(archs[0])


def read_config_json(model_dir: str) -> tuple[dict, dict | None]:
    path = os.path.join(model_dir, "config.json")
    if not os.path.exists(path):
        raise FileNotFoundError(f"{model_dir!r} has no config.json")
    with open(path, encoding="utf-8") as f:
        cfg = json.load(f)
    gen = None
    gpath = os.path.join(model_dir, "generation_config.json")
    if os.path.exists(gpath):
        with open(gpath, encoding="utf-8") as f:
            gen = json.load(f)
    return cfg, gen


def load_model_config(model_dir: str) -> ModelConfig:
    """``config.json`` (+ optional ``generation_config.json``) -> ``ModelConfig``."""
    cfg, gen = read_config_json(model_dir)
    return architecture_of(cfg).parse_config(cfg, gen)


def _load_builtin() -> None:
    if "Qwen2ForCausalLM" not in _ARCHITECTURES:
        from turingserve_b200.models import qwen2  # noqa: F401  (registers itself)
