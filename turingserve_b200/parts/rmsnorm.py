"""RMSNorm with the residual add fused in.

y = w * dtype(x32 * rsqrt(mean(x32^2) + eps)); with a residual, first residual = x + residual
(rounded to the model dtype) and the norm is taken of that sum
(turingserve/ops/reference.py:13-23, turingserve/ops/triton_rmsnorm.py:10-27).
"""

from __future__ import annotations

import torch

from turingserve_b200 import kernels
from turingserve_b200.parts.base import BuildContext, Norm, ParamSpec, register


class RMSNorm(Norm):
    def __init__(self, spec, ctx: BuildContext) -> None:
        self.eps = float(spec.eps)
        self.size = ctx.hidden_size
        self.weight: torch.Tensor | None = None

    def parameters(self) -> dict[str, ParamSpec]:
        return {"weight": ParamSpec((self.size,), compute_dtype=False, init="ones")}

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        self.weight = tensors["weight"].contiguous()

    def forward(self, x, residual: torch.Tensor | None = None) -> torch.Tensor:
        """``x`` is a tensor, or a product that its kernel left unreduced (it has shape, dtype and
        device; the norm kernel finishes the sum)."""
        out = torch.empty(x.shape, dtype=x.dtype, device=x.device)
        kernels.ops().rmsnorm(out, x, self.weight, self.eps, residual)
        return out


register("norm", "rmsnorm", RMSNorm)
