"""Rotary position encoding: per step, one table of cos/sin for every token and frequency.

angle(pos, i) = pos / theta^(2i / rot) for pair index i in [0, rot/2)
(``src/ops/kernels/cuda/rope_kernel.cu:102-123``, ``include/pulse/ops/kernels/rope_kernel.hpp:28-41``).
The reference recomputes pow/cos/sin per element and layer in 32-bit with fast-math; here the angle is
formed in 64-bit once per step and shared by all layers.  ``pairing`` says which elements of a head
form a pair: 'adjacent' (2i, 2i+1), as the reference rotates, or 'half' (i, i + rot/2).
"""
from __future__ import annotations

import torch

from .. import ops
from .base import PositionEncoding, register_part


@register_part("position_encoding", "rotary")
class RotaryEncoding(PositionEncoding):
    capturable = True       # see parts.base.Part.capturable
    def __init__(self, theta: float, rotary_dim: int, pairing: str = "adjacent"):
        if rotary_dim <= 0 or rotary_dim % 2:
            raise ValueError(f"rotary_dim must be positive and even, got {rotary_dim}")
        if pairing not in ("adjacent", "half"):
            raise ValueError(f"pairing must be 'adjacent' or 'half', got '{pairing}'")
        self.theta = float(theta)
        self.rotary_dim = rotary_dim
        self.pairing = pairing
        self._divisors: torch.Tensor | None = None

    def divisors(self, device) -> torch.Tensor:
        if self._divisors is None or self._divisors.device != device:
            pairs = self.rotary_dim // 2
            host = torch.tensor([self.theta ** (2.0 * i / self.rotary_dim) for i in range(pairs)], dtype=torch.float64)
            self._divisors = host.to(device)
        return self._divisors

    def prepare(self, ctx):
        cos, sin = ops.rope_table(ctx.positions, self.divisors(ctx.positions.device))
        return {"cos": cos, "sin": sin, "adjacent": self.pairing == "adjacent"}
