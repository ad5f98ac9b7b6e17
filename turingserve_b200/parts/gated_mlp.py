"""Dense gated feed-forward: down(silu(gate(x)) * up(x)), gate and up fused into one product
(turingserve/model/qwen2.py:35-36, turingserve/model/loader.py:84, turingserve/ops/reference.py:26-28).
"""

from __future__ import annotations

import torch

from turingserve_b200 import kernels
from turingserve_b200.parts.base import BuildContext, FeedForward, ParamSpec, register


class GatedMLP(FeedForward):
    def __init__(self, spec, ctx: BuildContext) -> None:
        if spec.activation != "silu":
            raise ValueError(f"gated_mlp: activation {spec.activation!r} has no kernel")
        self.hidden = ctx.hidden_size
        self.inter = int(spec.intermediate_size)
        self.bias = bool(spec.bias)
        self.w_gate_up = self.b_gate_up = self.w_down = self.b_down = None
        self.group = 0

    def parameters(self) -> dict[str, ParamSpec]:
        p = {"gate_proj.weight": ParamSpec((self.inter, self.hidden)),
             "up_proj.weight": ParamSpec((self.inter, self.hidden)),
             "down_proj.weight": ParamSpec((self.hidden, self.inter))}
        if self.bias:
            p["gate_proj.bias"] = ParamSpec((self.inter,))
            p["up_proj.bias"] = ParamSpec((self.inter,))
            p["down_proj.bias"] = ParamSpec((self.hidden,))
        return p

    # Gate and up rows are interleaved in blocks of GROUP when the width allows: a 128-row tile of the
    # fused product then holds 64 gates and their 64 ups, and a kernel that computes such a tile can
    # apply the activation before anything leaves the chip.
    GROUP = 64

    def _pack(self, gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
        if not self.group:
            return torch.cat([gate, up], dim=0).contiguous()
        g = gate.reshape(self.inter // self.group, self.group, *gate.shape[1:])
        u = up.reshape(self.inter // self.group, self.group, *up.shape[1:])
        return torch.cat([g, u], dim=1).reshape(2 * self.inter, *gate.shape[1:]).contiguous()

    def load(self, t: dict[str, torch.Tensor]) -> None:
        self.group = self.GROUP if self.inter % self.GROUP == 0 else 0
        self.w_gate_up = self._pack(t["gate_proj.weight"], t["up_proj.weight"])
        self.w_down = t["down_proj.weight"].contiguous()
        if self.bias:
            self.b_gate_up = self._pack(t["gate_proj.bias"], t["up_proj.bias"])
            self.b_down = t["down_proj.bias"].contiguous()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        ops = kernels.ops()
        T = x.shape[0]
        act = torch.empty((T, self.inter), dtype=x.dtype, device=x.device)
        ops.gated_linear(act, x, self.w_gate_up, self.b_gate_up, self.group)
        out = torch.empty((T, self.hidden), dtype=x.dtype, device=x.device)
        return ops.linear(out, act, self.w_down, self.b_down, may_defer=True)


register("feed_forward", "gated_mlp", GatedMLP)
