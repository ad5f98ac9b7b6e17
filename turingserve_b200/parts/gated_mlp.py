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

    def parameters(self) -> dict[str, ParamSpec]:
        p = {"gate_proj.weight": ParamSpec((self.inter, self.hidden)),
             "up_proj.weight": ParamSpec((self.inter, self.hidden)),
             "down_proj.weight": ParamSpec((self.hidden, self.inter))}
        if self.bias:
            p["gate_proj.bias"] = ParamSpec((self.inter,))
            p["up_proj.bias"] = ParamSpec((self.inter,))
            p["down_proj.bias"] = ParamSpec((self.hidden,))
        return p

    def load(self, t: dict[str, torch.Tensor]) -> None:
        self.w_gate_up = torch.cat([t["gate_proj.weight"], t["up_proj.weight"]], dim=0).contiguous()
        self.w_down = t["down_proj.weight"].contiguous()
        if self.bias:
            self.b_gate_up = torch.cat([t["gate_proj.bias"], t["up_proj.bias"]], dim=0).contiguous()
            self.b_down = t["down_proj.bias"].contiguous()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        ops = kernels.ops()
        T = x.shape[0]
        gu = torch.empty((T, 2 * self.inter), dtype=x.dtype, device=x.device)
        ops.linear(gu, x, self.w_gate_up, self.b_gate_up)
        act = torch.empty((T, self.inter), dtype=x.dtype, device=x.device)
        ops.silu_mul(act, gu)
        out = torch.empty((T, self.hidden), dtype=x.dtype, device=x.device)
        return ops.linear(out, act, self.w_down, self.b_down, may_defer=True)


register("feed_forward", "gated_mlp", GatedMLP)
