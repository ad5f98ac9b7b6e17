"""Rotate-half rotary position encoding: the fp32 cos/sin tables.

inv_freq[i] = 1 / theta**(2i/rotary_dim); angle = position * inv_freq, all in 32-bit
(turingserve/model/layers.py:13-18).  The rotation itself runs inside the kernel that also
writes keys and values to the cache; it uses the table rows cast to the model dtype and does
its arithmetic in 32-bit with one rounding (turingserve/ops/triton_rope.py:10-24).
"""

from __future__ import annotations

import torch

from turingserve_b200.parts.base import BuildContext, register


class RotaryEncoding:
    def __init__(self, spec, ctx: BuildContext) -> None:
        self.rotary_dim = int(spec.rotary_dim)
        self.theta = float(spec.theta)
        if self.rotary_dim % 2:
            raise ValueError("rotary_dim must be even")
        n = min(int(spec.max_positions), ctx.max_positions) if ctx.max_positions else int(spec.max_positions)
        self.max_positions = n
        inv_freq = 1.0 / (self.theta ** (torch.arange(0, self.rotary_dim, 2, dtype=torch.int64).float()
                                         / self.rotary_dim))
        freqs = torch.outer(torch.arange(n).float(), inv_freq)
        self.cos = freqs.cos().to(ctx.device).contiguous()
        self.sin = freqs.sin().to(ctx.device).contiguous()


register("position", "rope", RotaryEncoding)
