"""Dense gated feed-forward (SwiGLU): down(silu(gate(x)) * up(x)), no biases.

Reference parity: ``src/model/qwen3/model.cpp:893-916`` (three products, SiLU, elementwise product),
``src/ops/kernels/cuda/silu_kernel.cu:78-104`` (x / (1 + exp(-x)) in 32-bit).  Gate and up weights are
concatenated at load time so one product yields both; the activation and the product are one kernel with a
single rounding (the reference rounds after SiLU and again after the product).
"""
from __future__ import annotations

import torch

from .. import ops
from .base import FeedForward, TensorSpec, register_part


@register_part("feed_forward", "swiglu")
class SwiGLU(FeedForward):
    def __init__(self, hidden_size: int, intermediate_size: int):
        self.hidden_size = hidden_size
        self.intermediate_size = intermediate_size
        self.gate_up: torch.Tensor | None = None   # [2 * I, H]: gate rows, then up rows
        self.down: torch.Tensor | None = None      # [H, I]

    def tensor_specs(self) -> dict:
        h, i = self.hidden_size, self.intermediate_size
        return {"gate_proj.weight": TensorSpec((i, h)), "up_proj.weight": TensorSpec((i, h)),
                "down_proj.weight": TensorSpec((h, i))}

    def load(self, tensors: dict, runtime) -> None:
        gate, up = tensors["gate_proj.weight"], tensors["up_proj.weight"]
        if gate.dtype != up.dtype:
            up = up.to(gate.dtype)
        self.gate_up = torch.cat([gate, up], dim=0).contiguous()
        self.down = tensors["down_proj.weight"].contiguous()
        self._tensors = {"gate_up": self.gate_up, "down": self.down}

    def first_weights(self):
        return self.gate_up

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        gu = ops.linear(x, self.gate_up, ctx.act_dtype)
        act = ops.silu_mul(gu, prefetch=ctx.prefetch(self.down))
        return ops.linear(act, self.down, ctx.act_dtype)
