"""Typed description of a decoder model: which parts each layer is made of, and in which order
layers run.

A model is data: a tuple of ``LayerSpec`` (one per set of weights) and a tuple of ``LayerRun``
(the order in which those layers execute).  Every size and constant lives in a spec; the parts
under ``turingserve_b200.parts`` read them from there and nowhere else.

A spec is any frozen dataclass with a ``kind`` string; ``kind`` selects the implementation in
the part registries (``turingserve_b200.parts.registry``).  New kinds of mixer, feed-forward,
norm or position encoding bring their own spec class; nothing in this file lists them.

The reference keeps one flat ``Qwen2Config`` (turingserve/model/qwen2_config.py:10-63) and
hard-codes the layer recipe in ``Qwen2Model._run`` (turingserve/model/qwen2.py:38-61); here the
recipe itself is configuration so that layers of different kinds can alternate.
"""

from __future__ import annotations

from dataclasses import dataclass, fields, is_dataclass
from typing import Any


@dataclass(frozen=True)
class RMSNormSpec:
    """Root-mean-square norm over the last dimension with a learned scale."""

    eps: float
    kind: str = "rmsnorm"


@dataclass(frozen=True)
class RotarySpec:
    """Rotate-half rotary position encoding over the first ``rotary_dim`` dims of a head."""

    theta: float
    rotary_dim: int
    max_positions: int
    kind: str = "rope"


@dataclass(frozen=True)
class AttentionSpec:
    """Grouped-query softmax attention over a paged key/value cache.

    ``window`` = None means every earlier key is visible; an integer w means the query at
    position p sees keys at positions p-w+1 .. p.
    """

    num_heads: int
    num_kv_heads: int
    head_dim: int
    scale: float
    qkv_bias: bool
    out_bias: bool
    position: Any                       # a position-encoding spec, or None
    window: int | None = None
    kind: str = "attention"


@dataclass(frozen=True)
class GatedMLPSpec:
    """Dense gated feed-forward: down(act(gate(x)) * up(x))."""

    intermediate_size: int
    activation: str = "silu"
    bias: bool = False
    kind: str = "gated_mlp"


class LayerSpec:
    """One decoder layer: the spec of each of its parts under a ROLE name, and the arrangement that
    wires them.

    The roles are whatever the arrangement asks for.  "pre_norm" wants ``mixer``, ``feed_forward``,
    ``mixer_norm`` and ``ffn_norm``: ``h += mixer(norm(h)); h += ffn(norm(h))`` with the residual add
    deferred into the next norm (turingserve/model/qwen2.py:44-57).  An arrangement registered
    elsewhere may name others (a third norm, a second feed-forward); the same role names key the
    checkpoint prefixes in ``LayerTensorNames``.  A role's spec reads as an attribute: ``spec.mixer``.
    """

    def __init__(self, arrangement: str = "pre_norm", **roles: Any) -> None:
        if not roles:
            raise ValueError("a layer needs at least one part")
        object.__setattr__(self, "arrangement", arrangement)
        object.__setattr__(self, "roles", dict(roles))

    def __getattr__(self, role: str) -> Any:
        try:
            return self.__dict__["roles"][role]
        except KeyError:
            raise AttributeError(f"this layer has no part in role {role!r} (it has: "
                                 f"{', '.join(self.__dict__.get('roles', {}))})") from None

    def __setattr__(self, name: str, value: Any) -> None:
        raise AttributeError("LayerSpec is immutable")

    def __eq__(self, other: object) -> bool:
        return (isinstance(other, LayerSpec) and self.arrangement == other.arrangement
                and self.roles == other.roles)

    def __hash__(self) -> int:
        return hash((self.arrangement, tuple(sorted(self.roles))))

    def __repr__(self) -> str:
        inner = ", ".join(f"{k}={v!r}" for k, v in self.roles.items())
        return f"LayerSpec(arrangement={self.arrangement!r}, {inner})"


@dataclass(frozen=True)
class LayerRun:
    """One entry of the execution order.

    ``layer`` indexes ``ModelConfig.layers`` (the weights to use).  ``cache_from`` is None when
    this run owns a cache of its own, or the index of an EARLIER entry of the schedule whose
    cache this run reads without writing.
    """

    layer: int
    cache_from: int | None = None


@dataclass(frozen=True)
class ModelConfig:
    architecture: str
    hidden_size: int
    vocab_size: int
    layers: tuple[LayerSpec, ...]
    schedule: tuple[LayerRun, ...]
    final_norm: Any
    tie_word_embeddings: bool
    max_position_embeddings: int
    eos_token_ids: tuple[int, ...] = ()
    bos_token_id: int | None = None
    # constants of the architecture that no part's spec holds (what a model class registered with the
    # architecture reads: an embedding multiplier, a cap on the logits); plain data from config.json
    extras: tuple[tuple[str, Any], ...] = ()

    def extra(self, key: str, default: Any = None) -> Any:
        return dict(self.extras).get(key, default)

    def __post_init__(self) -> None:
        if not self.layers:
            raise ValueError("a model needs at least one layer")
        for r, run in enumerate(self.schedule):
            if not 0 <= run.layer < len(self.layers):
                raise ValueError(f"schedule[{r}] names layer {run.layer}, model has {len(self.layers)}")
            if run.cache_from is not None:
                if not 0 <= run.cache_from < r:
                    raise ValueError(f"schedule[{r}].cache_from={run.cache_from} must name an earlier run")
                if self.schedule[run.cache_from].cache_from is not None:
                    raise ValueError(f"schedule[{r}].cache_from={run.cache_from} names a run without a cache")

    @property
    def num_runs(self) -> int:
        return len(self.schedule)

    def run_layer(self, run_index: int) -> LayerSpec:
        return self.layers[self.schedule[run_index].layer]

    def with_schedule(self, schedule: list[LayerRun] | tuple[LayerRun, ...]) -> ModelConfig:
        kw = {f.name: getattr(self, f.name) for f in fields(self)}
        kw["schedule"] = tuple(schedule)
        return ModelConfig(**kw)


def spec_to_dict(spec: Any) -> Any:
    """Plain-data view of a spec tree (for logs and for the ``config`` key of the benchmark)."""
    if isinstance(spec, LayerSpec):
        return {"arrangement": spec.arrangement, **{k: spec_to_dict(v) for k, v in spec.roles.items()}}
    if is_dataclass(spec) and not isinstance(spec, type):
        return {f.name: spec_to_dict(getattr(spec, f.name)) for f in fields(spec)}
    if isinstance(spec, (tuple, list)):
        return [spec_to_dict(s) for s in spec]
    return spec
