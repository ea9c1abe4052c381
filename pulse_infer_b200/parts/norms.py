"""RMSNorm: x * rsqrt(mean(x^2) + eps) * w, computed in 32-bit, with the residual add fused in.

Reference parity: ``src/layer/rmsnorm.cpp:35-157`` and ``src/ops/kernels/cuda/rmsnorm_kernel.cu:97-118,147``
(eps inside the root; the weight multiplies directly, there is no ``1 + w``).
"""
from __future__ import annotations

import torch

from .. import ops
from .base import Norm, TensorSpec, register_part


@register_part("norm", "rmsnorm")
class RMSNorm(Norm):
    capturable = True       # see parts.base.Part.capturable
    def __init__(self, size: int, eps: float):
        self.size = size
        self.eps = float(eps)
        self.weight: torch.Tensor | None = None

    def tensor_specs(self) -> dict:
        return {"weight": TensorSpec((self.size,), init="ones_normal")}

    def load(self, tensors: dict, runtime) -> None:
        self.weight = tensors["weight"]
        self._tensors = {"weight": self.weight}

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        """x is a 32-bit residual [n, size]; returns the norm in the activation dtype."""
        return ops.add_rmsnorm(x, None, self.weight, self.eps, ctx.act_dtype)

    def add_norm(self, residual: torch.Tensor, delta, ctx, rows=None, upcoming=None) -> torch.Tensor:
        return ops.add_rmsnorm(residual, delta, self.weight, self.eps, ctx.act_dtype, rows=rows,
                               prefetch=ctx.prefetch(upcoming))

    def fusable(self):
        return self.weight, self.eps
