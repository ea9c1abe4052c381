"""Grouped-query attention over the paged cache, with optional per-head RMSNorm of queries and keys,
an optional position encoding applied to both, and an optional window.

Reference parity: ``src/model/qwen3/model.cpp:779-879`` - q/k/v projections without bias, per-head
RMSNorm over the head size with one weight shared by all heads and the layer's eps, rotation of
queries and keys, keys (rotated) and values (raw) written to the pages of the token's request before
any query of the step attends, scores scaled by 1/sqrt(head size), causal by absolute position,
kv head = head / (heads / kv heads), output projection without bias.
The three projections are one product here (weights concatenated at load time); norm, rotation and the
page write are one kernel.
"""
from __future__ import annotations

import math

import torch

from .. import ops
from .base import CacheSpec, Mixer, TensorSpec, register_part


@register_part("mixer", "attention")
class Attention(Mixer):
    capturable = True       # see parts.base.Part.capturable
    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, qk_norm: bool = True,
                 norm_eps: float = 1e-6, position: str | None = "rotary", window: int | None = None,
                 scale: float | None = None, writes_cache: bool = True):
        if num_heads % num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        self.hidden_size = hidden_size
        self.num_heads = num_heads
        self.num_kv_heads = num_kv_heads
        self.head_dim = head_dim
        self.qk_norm = qk_norm
        self.norm_eps = float(norm_eps)
        self.position = position            # name of the position encoding whose tables to use, or None
        self.window = window
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)
        # False: this layer projects no keys or values and attends over a cache another layer fills
        self.writes_cache = writes_cache
        self.qkv: torch.Tensor | None = None
        self.o: torch.Tensor | None = None
        self.q_norm: torch.Tensor | None = None
        self.k_norm: torch.Tensor | None = None

    @property
    def q_size(self) -> int:
        return self.num_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_kv_heads * self.head_dim

    def cache_spec(self) -> CacheSpec:
        return CacheSpec(self.num_kv_heads, self.head_dim, self.window)

    def uses_key_ranges(self, page_size: int, act_dtype: torch.dtype) -> bool:
        """Whether decode steps of this layer cut each request's keys into ranges whose number must be bounded when a
        step is recorded (the mma.sync decode kernel); the tcgen05 decode kernel divides the step's keys by itself."""
        return not ops.decode_on_tcgen05(self.head_dim, page_size, self.num_heads // self.num_kv_heads, act_dtype)

    def tensor_specs(self) -> dict:
        specs = {"q_proj.weight": TensorSpec((self.q_size, self.hidden_size)),
                 "o_proj.weight": TensorSpec((self.hidden_size, self.q_size))}
        if self.writes_cache:
            specs["k_proj.weight"] = TensorSpec((self.kv_size, self.hidden_size))
            specs["v_proj.weight"] = TensorSpec((self.kv_size, self.hidden_size))
        if self.qk_norm:
            specs["q_norm.weight"] = TensorSpec((self.head_dim,), init="ones_normal")
            if self.writes_cache:
                specs["k_norm.weight"] = TensorSpec((self.head_dim,), init="ones_normal")
        return specs

    def load(self, tensors: dict, runtime) -> None:
        q = tensors["q_proj.weight"]
        if self.writes_cache:
            parts = [q, tensors["k_proj.weight"].to(q.dtype), tensors["v_proj.weight"].to(q.dtype)]
            self.qkv = torch.cat(parts, dim=0).contiguous()
        else:
            self.qkv = q.contiguous()
        self.o = tensors["o_proj.weight"].contiguous()
        if self.qk_norm:
            self.q_norm = tensors["q_norm.weight"]
            self.k_norm = tensors["k_norm.weight"].to(self.q_norm.dtype) if self.writes_cache else None
        self._tensors = {"qkv": self.qkv, "o": self.o}
        self.attention_impl = getattr(runtime, "attention_impl", "auto")

    def first_weights(self):
        return self.qkv

    takes_deferred_norm = True
    adds_to_residual = True

    def forward(self, x, ctx, cache, residual: torch.Tensor | None = None, next_norm=None):
        """x [T, H] in the activation dtype (or ``ops.NormedRows``: a norm that the first product finishes);
        ``cache`` is the view of this execution's cache (key pool, value pool, block table of its group).
        With ``residual`` the output product may add its result there and return None, or the input it
        prepared for ``next_norm``."""
        nkv_written = self.num_kv_heads if self.writes_cache else 0
        qkv = ops.linear(x, self.qkv, ctx.act_dtype)
        rot = ctx.position_data.get(self.position) if self.position else None
        use_mma = (ctx.act_dtype == torch.bfloat16 and self.attention_impl != "simple"
                   and self.head_dim % 16 == 0 and self.head_dim <= 256)
        if use_mma and self.writes_cache and ctx.has_decode and not ctx.has_prompt and qkv.is_contiguous():
            # a step of single tokens: per-head norm, rotation and the page write happen inside the attention kernel
            scratch = ctx.attention_scratch(self.num_heads, self.head_dim, self.window, self.num_kv_heads)
            if scratch.decode_ws is not None and ops.attention_decode_fused_usable(
                    self.head_dim, cache.page_size, self.num_heads // self.num_kv_heads, rot["adjacent"] if rot else True,
                    ctx.act_dtype):
                attn = ops.attention_decode_fused(
                    qkv, cache.keys, cache.values, cache.block_table, ctx.seg_off, ctx.seg_slot, ctx.seg_start, ctx.seg_len,
                    ctx.num_segments, self.num_heads, self.num_kv_heads, self.head_dim, cache.page_size, self.window,
                    self.scale, self.q_norm, self.k_norm, self.norm_eps, rot["cos"] if rot else None,
                    rot["sin"] if rot else None, ctx.error_count, workspace=scratch.decode_ws)
                return ops.linear(attn, self.o, ctx.act_dtype, residual=residual, next_norm=next_norm)
        ops.qk_norm_rope_write(
            qkv, self.q_norm, self.k_norm, self.norm_eps,
            rot["cos"] if rot else None, rot["sin"] if rot else None, rot["adjacent"] if rot else True,
            cache.keys, cache.values, cache.block_table, ctx.token_slot, ctx.positions, cache.page_size,
            self.num_heads, nkv_written, self.head_dim, ctx.error_count, prefetch=ctx.prefetch(self.o))
        q_stride = qkv.shape[1]
        if use_mma:
            scratch = ctx.attention_scratch(self.num_heads, self.head_dim, self.window, self.num_kv_heads)
            attn = ops.attention_mma(
                qkv, q_stride, cache.keys, cache.values, cache.block_table, ctx.seg_off, ctx.seg_slot, ctx.seg_start,
                ctx.seg_len, ctx.token_seg, ctx.num_tokens, ctx.num_segments, ctx.max_seg_len, ctx.has_prompt,
                ctx.has_decode, scratch.max_splits, scratch.acc, scratch.ml, self.num_heads, self.num_kv_heads,
                self.head_dim, cache.page_size, self.window, self.scale, split_keys=scratch.split_keys,
                prefetch=ctx.prefetch(getattr(ctx, "upcoming_weights", None)), prompt_splits=scratch.prompt_splits,
                prompt_acc=scratch.prompt_acc, prompt_ml=scratch.prompt_ml, decode_ws=scratch.decode_ws,
                decode_on_tcgen05=scratch.decode_ws is not None)
        else:
            attn = ops.attention_simple(
                qkv, q_stride, cache.keys, cache.values, cache.block_table, ctx.token_slot, ctx.positions,
                ctx.num_tokens, self.num_heads, self.num_kv_heads, self.head_dim, cache.page_size, self.window,
                self.scale)
        return ops.linear(attn, self.o, ctx.act_dtype, residual=residual, next_norm=next_norm)
