"""Interfaces of the parts a model is put together from, and the registries that map a kind to a class.

A part receives every size and constant as a constructor parameter, declares the tensors it wants
(names relative to its prefix, with shapes) and is handed them once at load time.  No part knows
which model it sits in.  The five families:

* ``Mixer``            mixes information across positions (attention here).  ``forward(x, ctx, cache)``.
                       Declares what it needs from the cache manager: token pages (``CacheSpec``) and/or
                       fixed-size per-request state (``StateSpec``).
* ``FeedForward``      position-wise transformation (dense SwiGLU here).  ``forward(x, ctx)``.
* ``Norm``             ``forward(x)`` and the fused ``add_norm(residual, delta, rows=None)``.
* ``PositionEncoding`` ``prepare(ctx)`` computes whatever the step needs once (rotation tables).
* ``Block``            wires two norms, a mixer and a feed-forward around the residual stream.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch


@dataclass(frozen=True)
class TensorSpec:
    """A tensor a part wants.  ``init`` tells the random-weights mode how to fill it:
    'normal' = N(0, 0.02), 'ones_normal' = 1 + N(0, 0.02)."""
    shape: tuple
    init: str = "normal"
    optional: bool = False


@dataclass(frozen=True)
class CacheSpec:
    """Token pages a mixer needs: keys and values per token.  Layers whose specs are equal share a
    page group (one block table, one page id addressing the same slot in each of their pools)."""
    num_kv_heads: int
    head_dim: int
    window: int | None = None     # None: all keys are kept; n: only the last n keys are ever read


@dataclass(frozen=True)
class StateSpec:
    """Fixed-size state a mixer keeps per request, independent of the number of tokens."""
    shape: tuple
    dtype: torch.dtype = torch.float32


class Part:
    kind: str = ""
    # True: ``forward`` may be recorded once into a CUDA graph and replayed for later steps of the same shape.  A part
    # that says so promises that its forward (1) takes everything that changes from step to step - tokens, positions,
    # slots, segment starts and lengths - from the device tensors of ``ctx``, never from host values such as
    # ``ctx.segments`` or a Python loop over requests, (2) launches the same kernels with the same arguments for every
    # step of that shape, and (3) may run twice on one step's data (a warm-up before the recording) without harm:
    # whatever it writes is idempotent (pages) or lives in ``cache.state``, which the engine puts back after the
    # warm-up.  The default is False: a step whose model holds such a part is launched kernel by kernel.
    capturable: bool = False

    def tensor_specs(self) -> dict:
        """name (relative to the part's prefix) -> TensorSpec."""
        return {}

    def load(self, tensors: dict, runtime) -> None:
        """Receive the tensors named by ``tensor_specs`` (already on the device, in the dtype the
        loading policy gives them).  Optional tensors that the file lacks are absent."""

    def num_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in getattr(self, "_tensors", {}).values())

    def first_weights(self):
        """The weight tensor this part's forward streams first, if any: the kernel that runs just before
        it may ask the L2 to start fetching it (see ``StepContext.prefetch``)."""
        return None


class Mixer(Part):
    # Two optional abilities that a block makes use of when a part declares them:
    # takes_deferred_norm: forward() accepts ``ops.NormedRows`` for x (a norm that the first product finishes itself)
    # adds_to_residual: forward(..., residual=h, next_norm=(weight, eps, owner) or None) may add its output to the
    #     float32 residual h itself; it then returns None, or the ``ops.NormedRows`` prepared for ``next_norm``
    takes_deferred_norm = False
    adds_to_residual = False

    def cache_spec(self) -> CacheSpec | None:
        return None

    def state_spec(self) -> StateSpec | None:
        return None

    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    takes_deferred_norm = False      # as for mixers
    adds_to_residual = False

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        raise NotImplementedError


class Norm(Part):
    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        raise NotImplementedError

    def add_norm(self, residual: torch.Tensor, delta: torch.Tensor | None, ctx, rows: torch.Tensor | None = None,
                 upcoming=None):
        """residual (fp32, updated in place unless ``rows`` is given) += delta; returns norm(residual).
        ``upcoming``: weights the next product will stream (a prefetch hint, may be ignored)."""
        raise NotImplementedError

    def fusable(self):
        """(weight, eps) if this norm is x * rsqrt(mean(x^2) + eps) * weight, so that the products around it can
        prepare and finish it (see ``ops.NormedRows``); None otherwise (the default)."""
        return None


class PositionEncoding(Part):
    def prepare(self, ctx):
        """Called once per step before the layers run; returns what mixers read from ``ctx.position_data``."""
        return None


class Block(Part):
    def forward(self, stream, ctx, cache) -> None:
        raise NotImplementedError

    def first_norm(self):
        """The norm this block applies to the stream first, if it starts with one (a hint for the block before)."""
        return None


@dataclass
class ResidualStream:
    """The residual sum, kept in 32-bit, with the last sub-layer's output not yet added: the add is
    fused into the next norm (or into the final gather)."""
    hidden: torch.Tensor                 # fp32 [T, H]
    pending: torch.Tensor | None = None  # [T, H] activation dtype
    prepared: object | None = None       # ops.NormedRows: the next norm's input, made by the product that added last
    next_norm: object | None = None      # the norm that the next block applies first (set by the model's loop)


# ---- registries -----------------------------------------------------------------------------------
MIXERS: dict[str, type] = {}
FEED_FORWARDS: dict[str, type] = {}
NORMS: dict[str, type] = {}
POSITION_ENCODINGS: dict[str, type] = {}
BLOCKS: dict[str, type] = {}
EMBEDDINGS: dict[str, type] = {}
HEADS: dict[str, type] = {}
_FAMILIES = {"mixer": MIXERS, "feed_forward": FEED_FORWARDS, "norm": NORMS,
             "position_encoding": POSITION_ENCODINGS, "block": BLOCKS, "embedding": EMBEDDINGS, "head": HEADS}


def register_part(family: str, kind: str, replace: bool = False):
    """Class decorator: ``@register_part('mixer', 'attention')``."""
    table = _FAMILIES[family]

    def deco(cls):
        if kind in table and not replace:
            raise ValueError(f"{family} kind '{kind}' is already registered")
        cls.kind = kind
        table[kind] = cls
        return cls
    return deco


def build_part(family: str, kind: str, params: dict):
    table = _FAMILIES[family]
    if kind not in table:
        raise KeyError(f"unknown {family} kind '{kind}'; known: {', '.join(sorted(table))}")
    return table[kind](**params)
