"""Interfaces of the model's parts and the registries that choose an implementation by
``spec.kind``.

A part knows its own sizes (from its spec) and nothing about the model it sits in.  The model
hands each part its tensors by LOCAL name (e.g. ``q_proj.weight``); which checkpoint prefix those
live under is the architecture's business (``turingserve_b200.config.registry.TensorNames``).

Interfaces
----------
Norm            forward(x, residual=None) -> y          (residual updated in place when given; x may be a
                                                         product left unreduced by its kernel, which a
                                                         norm either passes to a kernel that finishes it
                                                         or turns into a tensor with ops().materialize)
PositionEncoding  tables()/apply are private to the mixers that accept it
Mixer           forward(x, step, cache, state) -> y     cache_need() / state_need() declare memory
FeedForward     forward(x) -> y                         (mixers and feed-forwards get tensors; they may
                                                         return what ops().linear(..., may_defer=True) gave)
Block           forward(h, residual, step, cache, state) -> (h, residual)

``step`` is a ``StepInputs`` (turingserve_b200.engine.batch): the flat batch on the device.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable

import torch


@dataclass(frozen=True)
class ParamSpec:
    """One checkpoint tensor a part reads.

    ``compute_dtype`` True: converted to the engine's dtype (operands of matrix products,
    embeddings).  False: a tensor stored in 32 bits stays in 32 bits, anything else is converted.
    ``integer`` True: an integer table, kept as int32.
    """

    shape: tuple[int, ...]
    compute_dtype: bool = True
    integer: bool = False
    init: str = "normal"            # "normal" | "ones" | "zeros": how the random-weights mode fills it


@dataclass(frozen=True)
class CacheNeed:
    """What a mixer wants from the paged cache: keys and values of ``num_kv_heads`` x ``head_dim``
    per token; ``window`` None keeps every token, an integer keeps the last ``window`` of them."""

    num_kv_heads: int
    head_dim: int
    window: int | None = None


@dataclass(frozen=True)
class StateNeed:
    """Fixed-size per-request state of a mixer (zeroed when a request is admitted)."""

    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32


class Part:
    """Base of all parts: declares parameters, receives them."""

    def parameters(self) -> dict[str, ParamSpec]:
        return {}

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        """Receive the tensors named by ``parameters()``, already on the device and converted."""
        if tensors:
            raise ValueError(f"{type(self).__name__} takes no tensors, got {sorted(tensors)}")


class Norm(Part):
    def forward(self, x: torch.Tensor, residual: torch.Tensor | None = None) -> torch.Tensor:
        raise NotImplementedError


class Mixer(Part):
    def cache_need(self) -> CacheNeed | None:
        return None

    def state_need(self) -> StateNeed | None:
        return None

    def forward(self, x: torch.Tensor, step, cache, state: torch.Tensor | None) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


@dataclass(frozen=True)
class BuildContext:
    """What every part constructor gets besides its spec."""

    hidden_size: int
    dtype: torch.dtype
    device: torch.device
    max_positions: int              # longest sequence the engine will run (sizes position tables)


_REGISTRIES: dict[str, dict[str, Callable[[Any, BuildContext], Any]]] = {
    "norm": {}, "position": {}, "mixer": {}, "feed_forward": {}, "block": {},
}


def register(family: str, kind: str, factory: Callable[[Any, BuildContext], Any]) -> None:
    """Register ``factory(spec, ctx) -> part`` for ``spec.kind == kind`` in ``family``
    (norm | position | mixer | feed_forward | block)."""
    _REGISTRIES[family][kind] = factory


def build(family: str, spec: Any, ctx: BuildContext):
    _load_builtin()
    kind = spec if isinstance(spec, str) else getattr(spec, "kind", None)
    try:
        factory = _REGISTRIES[family][kind]
    except KeyError:
        known = ", ".join(sorted(_REGISTRIES[family])) or "none"
        raise ValueError(f"no {family} registered for kind {kind!r} (registered: {known})") from None
    return factory(spec, ctx)


_loaded = False


def _load_builtin() -> None:
    global _loaded
    if not _loaded:
        _loaded = True
        from turingserve_b200.parts import attention, block, gated_mlp, rmsnorm, rotary  # noqa: F401


def build_block(layer_spec: Any, ctx: BuildContext):
    """Build one layer; ``layer_spec.arrangement`` chooses the wiring."""
    _load_builtin()
    try:
        factory = _REGISTRIES["block"][layer_spec.arrangement]
    except KeyError:
        known = ", ".join(sorted(_REGISTRIES["block"])) or "none"
        raise ValueError(f"no block arrangement {layer_spec.arrangement!r} (registered: {known})") from None
    return factory(layer_spec, ctx)
