"""Dense gated feed-forward (SwiGLU): down(silu(gate(x)) * up(x)), no biases.

Reference parity: ``src/model/qwen3/model.cpp:893-916`` (three products, SiLU, elementwise product),
``src/ops/kernels/cuda/silu_kernel.cu:78-104`` (x / (1 + exp(-x)) in 32-bit).  Gate and up weights are
joined at load time so one product yields both; the activation and the product are one kernel with a
single rounding (the reference rounds after SiLU and again after the product).  When the intermediate size
is a multiple of 16 the joined rows are interleaved in blocks of 16 gate / 16 up features: portions of more than
a few tokens then run on the tcgen05 product whose epilogue applies SiLU(gate) * up straight from tensor memory,
so the [T, 2I] intermediate is never written.
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
        self.gate_up: torch.Tensor | None = None   # [2 * I, H]: gate and up rows, blocked by 16 or gate-then-up
        self.down: torch.Tensor | None = None      # [H, I]
        self.blocked = False

    def tensor_specs(self) -> dict:
        h, i = self.hidden_size, self.intermediate_size
        return {"gate_proj.weight": TensorSpec((i, h)), "up_proj.weight": TensorSpec((i, h)),
                "down_proj.weight": TensorSpec((h, i))}

    def load(self, tensors: dict, runtime) -> None:
        gate, up = tensors["gate_proj.weight"], tensors["up_proj.weight"]
        if gate.dtype != up.dtype:
            up = up.to(gate.dtype)
        self.blocked = self.intermediate_size % 16 == 0
        self.gate_up = ops.interleave_gate_up(gate, up) if self.blocked else torch.cat([gate, up], dim=0).contiguous()
        self.down = tensors["down_proj.weight"].contiguous()
        self._tensors = {"gate_up": self.gate_up, "down": self.down}

    def first_weights(self):
        return self.gate_up

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        if (self.blocked and self.gate_up.dtype == torch.bfloat16 and x.dtype == torch.bfloat16
                and x.shape[0] > ops.kernels.SMALL_M_ROWS and self.hidden_size % 8 == 0):
            act = ops.gemm_tcgen05(x, self.gate_up, torch.bfloat16, gated=True)      # product + SiLU * up in one kernel
        else:
            gu = ops.linear(x, self.gate_up, ctx.act_dtype)
            act = ops.silu_mul(gu, prefetch=ctx.prefetch(self.down), blocked=self.blocked)
        return ops.linear(act, self.down, ctx.act_dtype)
