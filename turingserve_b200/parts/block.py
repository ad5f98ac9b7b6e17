"""How a mixer, a feed-forward and their norms are wired into one layer.

"pre_norm" carries (h, residual) and defers each residual add into the next norm: the first
block takes residual = h; afterwards every norm first does residual = h + residual in the model
dtype (turingserve/model/qwen2.py:42-57).
"""

from __future__ import annotations

from turingserve_b200.parts.base import BuildContext, build, register


class PreNormBlock:
    def __init__(self, spec, ctx: BuildContext) -> None:
        self.mixer_norm = build("norm", spec.mixer_norm, ctx)
        self.mixer = build("mixer", spec.mixer, ctx)
        self.ffn_norm = build("norm", spec.ffn_norm, ctx)
        self.feed_forward = build("feed_forward", spec.feed_forward, ctx)

    def parts(self) -> dict[str, object]:
        """Sub-parts by the role names used in ``LayerTensorNames``."""
        return {"mixer_norm": self.mixer_norm, "mixer": self.mixer,
                "ffn_norm": self.ffn_norm, "feed_forward": self.feed_forward}

    def forward(self, h, residual, step, cache, state):
        if residual is None:
            residual = h
            x = self.mixer_norm.forward(h)
        else:
            x = self.mixer_norm.forward(h, residual)
        a = self.mixer.forward(x, step, cache, state)
        x = self.ffn_norm.forward(a, residual)
        h = self.feed_forward.forward(x)
        return h, residual


def _build_block(spec, ctx: BuildContext):
    return PreNormBlock(spec, ctx)


register("block", "pre_norm", _build_block)
