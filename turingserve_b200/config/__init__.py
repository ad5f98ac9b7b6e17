"""Typed configuration: model description, engine options, architecture registry."""

from turingserve_b200.config.engine_config import EngineConfig
from turingserve_b200.config.model_config import (
    AttentionSpec, GatedMLPSpec, LayerRun, LayerSpec, ModelConfig, RMSNormSpec, RotarySpec)
from turingserve_b200.config.registry import (
    Architecture, LayerTensorNames, TensorNames, architecture_of, get_architecture,
    load_model_config, register_architecture)

__all__ = [
    "EngineConfig", "AttentionSpec", "GatedMLPSpec", "LayerRun", "LayerSpec", "ModelConfig",
    "RMSNormSpec", "RotarySpec", "Architecture", "LayerTensorNames", "TensorNames",
    "architecture_of", "get_architecture", "load_model_config", "register_architecture",
]
