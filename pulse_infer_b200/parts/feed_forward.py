"""Dense gated feed-forward (SwiGLU): down(silu(gate(x)) * up(x)), no biases.

Reference parity: ``src/model/qwen3/model.cpp:893-916`` (three products, SiLU, elementwise product),
``src/ops/kernels/cuda/silu_kernel.cu:78-104`` (x / (1 + exp(-x)) in 32-bit).  Gate and up weights are
joined at load time so one product yields both; the activation and the product are one kernel with a
single rounding (the reference rounds after SiLU and again after the product).  When the intermediate size
is a multiple of 8 the joined rows are interleaved in blocks of 8 gate / 8 up features, and in bfloat16 the
activation is the epilogue of the product, so the [T, 2I] intermediate is never written: portions of more than
a few tokens run on the tcgen05 product, which applies SiLU(gate) * up straight from tensor memory; a few
rows (decoding) run on the weight-streaming product, whose 16-row tiles then hold gate and up of 8 features.
"""
from __future__ import annotations

import torch

from .. import ops
from .base import FeedForward, TensorSpec, register_part


@register_part("feed_forward", "swiglu")
class SwiGLU(FeedForward):
    capturable = True       # see parts.base.Part.capturable
    def __init__(self, hidden_size: int, intermediate_size: int):
        self.hidden_size = hidden_size
        self.intermediate_size = intermediate_size
        self.gate_up: torch.Tensor | None = None   # [2 * I, H]: gate and up rows, in blocks of 8 or gate-then-up
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
        self.blocked = self.intermediate_size % ops.kernels.GATE_BLOCK == 0
        self.gate_up = ops.interleave_gate_up(gate, up) if self.blocked else torch.cat([gate, up], dim=0).contiguous()
        self.down = tensors["down_proj.weight"].contiguous()
        self._tensors = {"gate_up": self.gate_up, "down": self.down}

    def first_weights(self):
        return self.gate_up

    takes_deferred_norm = True
    adds_to_residual = True

    def forward(self, x, ctx, residual: torch.Tensor | None = None, next_norm=None):
        """With ``residual`` the down product may add its result there and return None, or the input it prepared
        for ``next_norm``."""
        if isinstance(x, ops.NormedRows):
            sc = x.scaled
            if x._value is None and self.blocked and ops.small_m_usable(sc.shape[0], sc.shape[1], self.gate_up):
                # the norm's scale, both products and SiLU * up in one kernel
                act = ops.gemm_small_m(sc, self.gate_up, torch.bfloat16, gated=True, row_ssq=(x.partials, x.eps))
                return ops.linear(act, self.down, ctx.act_dtype, residual=residual, next_norm=next_norm)
            x = x.materialize()
        fused = (self.blocked and self.gate_up.dtype == torch.bfloat16 and x.dtype == torch.bfloat16
                 and self.hidden_size % 8 == 0 and x.stride(-1) == 1 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0)
        if fused and x.shape[0] > ops.kernels.SMALL_M_ROWS:
            act = ops.gemm_tcgen05(x, self.gate_up, torch.bfloat16, gated=True)      # product + SiLU * up in one kernel
        elif fused and ops.small_m_usable(x.shape[0], self.hidden_size, self.gate_up):
            act = ops.gemm_small_m(x, self.gate_up, torch.bfloat16, gated=True)      # the same for a few rows
        else:
            gu = ops.linear(x, self.gate_up, ctx.act_dtype)
            act = ops.silu_mul(gu, prefetch=ctx.prefetch(self.down), blocked=self.blocked)
        return ops.linear(act, self.down, ctx.act_dtype, residual=residual, next_norm=next_norm)
