"""Model parts: norm, position encoding, mixer, feed-forward, block, and the decoder built of them."""

from turingserve_b200.parts.base import (
    BuildContext, CacheNeed, FeedForward, Mixer, Norm, ParamSpec, Part, StateNeed, build,
    build_block, register)

__all__ = ["BuildContext", "CacheNeed", "FeedForward", "Mixer", "Norm", "ParamSpec", "Part",
           "StateNeed", "build", "build_block", "register"]
