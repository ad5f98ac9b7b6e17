"""What a request asks of the sampler and of the finish rules.

The option names are the ones users of the reference know (its ``SamplingParams``,
turingserve/engine/sampling_params.py:8-30), because requests written for it should read the same
here; ``stop`` strings have no counterpart, since this engine sees token ids only.  The limits are
kept in one table and checked in one loop; an option outside its limits names itself, its value
and the interval in the error.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field

# option -> (lowest, highest, lowest allowed itself?, highest allowed itself?)
_LIMITS: dict[str, tuple[float, float, bool, bool]] = {
    "temperature": (0.0, 2.0, True, True),
    "top_p": (0.0, 1.0, False, True),
    "max_tokens": (1, math.inf, True, False),
    "repetition_penalty": (0.0, math.inf, False, False),
    "presence_penalty": (-2.0, 2.0, True, True),
    "frequency_penalty": (-2.0, 2.0, True, True),
}
_GREEDY_BELOW = 1e-5        # a temperature this small means "take the best token"
_NO_TOP_K = -1


def _interval(lo: float, hi: float, lo_in: bool, hi_in: bool) -> str:
    left = ("[" if lo_in else "(") + ("-inf" if lo == -math.inf else f"{lo:g}")
    right = ("inf" if hi == math.inf else f"{hi:g}") + ("]" if hi_in else ")")
    return f"{left}, {right}"


@dataclass
class SamplingParams:
    # how long
    max_tokens: int = 16
    min_tokens: int = 0                 # stop tokens cannot be drawn before this many were produced
    stop_token_ids: list[int] = field(default_factory=list)
    ignore_eos: bool = False
    # how to draw
    temperature: float = 1.0
    top_k: int = _NO_TOP_K              # keep the k most likely tokens; -1 keeps all
    top_p: float = 1.0                  # keep the smallest set of tokens with this much probability
    seed: int | None = None             # None: derived from the engine's seed and the arrival number
    # what to discourage
    repetition_penalty: float = 1.0
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0

    def __post_init__(self) -> None:
        for name, (lo, hi, lo_in, hi_in) in _LIMITS.items():
            v = getattr(self, name)
            inside = (v > lo or (lo_in and v == lo)) and (v < hi or (hi_in and v == hi))
            if not inside:
                raise ValueError(f"{name}={v!r} is outside {_interval(lo, hi, lo_in, hi_in)}")
        if self.top_k != _NO_TOP_K and self.top_k <= 0:
            raise ValueError(f"top_k={self.top_k!r}: a positive count, or {_NO_TOP_K} to keep every token")
        if not 0 <= self.min_tokens <= self.max_tokens:
            raise ValueError(f"min_tokens={self.min_tokens!r} does not lie between 0 and max_tokens={self.max_tokens!r}")

    @property
    def greedy(self) -> bool:
        return self.temperature < _GREEDY_BELOW

    @property
    def uses_penalties(self) -> bool:
        neutral = (1.0, 0.0, 0.0)
        return (self.repetition_penalty, self.presence_penalty, self.frequency_penalty) != neutral

    @property
    def filters(self) -> bool:
        return self.top_k != _NO_TOP_K or self.top_p < 1.0
