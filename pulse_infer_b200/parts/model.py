"""The generic decoder: builds the parts a ``ModelSpec`` names and runs them in the order it lists.

It is the only model class; an architecture contributes a configuration and a spec builder, never
code in here.  ``forward(ctx)`` runs exactly the tokens of the step and returns 32-bit logits at the
wanted rows (the reference computes the final norm and the head on every row,
``src/model/qwen3/model.cpp:1305-1344``).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..models.spec import ModelSpec
from .base import ResidualStream, build_part


@dataclass
class Runtime:
    """Where and how the model computes.  ``mode`` 'bfloat16': bf16 activations, pages and products
    with 32-bit accumulation; 'float32': everything in true 32-bit."""
    device: torch.device
    mode: str = "bfloat16"
    attention_impl: str = "auto"     # 'auto' (tensor-core kernel in bfloat16) or 'simple'

    def __post_init__(self):
        self.device = torch.device(self.device)
        if self.mode in ("bf16",):
            self.mode = "bfloat16"
        if self.mode in ("fp32", "f32"):
            self.mode = "float32"
        if self.mode not in ("bfloat16", "float32"):
            raise ValueError(f"dtype must be 'bfloat16' or 'float32', got '{self.mode}'")

    @property
    def act_dtype(self) -> torch.dtype:
        return torch.bfloat16 if self.mode == "bfloat16" else torch.float32


class DecoderModel:
    def __init__(self, spec: ModelSpec, runtime: Runtime):
        self.spec = spec
        self.runtime = runtime
        self.embedding = build_part("embedding", spec.embedding.kind, spec.embedding.params)
        self.positions = {name: build_part("position_encoding", ps.kind, ps.params)
                          for name, ps in spec.positions.items()}
        self.layers = []
        for ls in spec.layers:
            mixer = build_part("mixer", ls.mixer.kind, ls.mixer.params)
            ff = build_part("feed_forward", ls.feed_forward.kind, ls.feed_forward.params)
            n1 = build_part("norm", ls.mixer_norm.kind, ls.mixer_norm.params)
            n2 = build_part("norm", ls.feed_forward_norm.kind, ls.feed_forward_norm.params)
            self.layers.append(build_part("block", ls.arrangement, dict(mixer=mixer, feed_forward=ff,
                                                                       mixer_norm=n1, feed_forward_norm=n2)))
        self.final_norm = build_part("norm", spec.final_norm.kind, spec.final_norm.params)
        self.lm_head = build_part("head", spec.lm_head.kind, spec.lm_head.params)
        self.order = tuple(spec.order)
        for entry in self.order:
            if not (0 <= entry.layer < len(self.layers)):
                raise ValueError(f"schedule names layer {entry.layer}, the model has {len(self.layers)}")
        self._check_caches()

    # ---- what the cache manager must provide -------------------------------------------------------
    def _check_caches(self) -> None:
        specs: dict[int, object] = {}
        writers: set[int] = set()
        for entry in self.order:
            mixer = self.layers[entry.layer].mixer
            cs = mixer.cache_spec()
            if cs is None:
                continue
            if entry.cache is None:
                raise ValueError(f"layer {entry.layer} needs token pages but its schedule entry names no cache")
            if entry.cache in specs and specs[entry.cache] != cs:
                raise ValueError(f"cache {entry.cache} is used by layers with different needs")
            specs[entry.cache] = cs
            if getattr(mixer, "writes_cache", True):
                if entry.cache in writers:
                    raise ValueError(f"cache {entry.cache} is written by two schedule entries")
                writers.add(entry.cache)
            elif entry.cache not in writers:
                raise ValueError(f"layer {entry.layer} reads cache {entry.cache} before any entry has written it")
        self._cache_specs = [specs.get(i) for i in range(self.spec.num_caches)]

    def cache_specs(self) -> list:
        return list(self._cache_specs)

    def state_specs(self) -> list:
        return [layer.mixer.state_spec() for layer in self.layers]

    def all_parts(self):
        """Every part of the model, the blocks and what they are made of included."""
        yield self.embedding
        yield from self.positions.values()
        for block in self.layers:
            yield block
            for name in ("mixer", "feed_forward", "mixer_norm", "feed_forward_norm"):
                part = getattr(block, name, None)
                if part is not None:
                    yield part
        yield self.final_norm
        yield self.lm_head

    @property
    def capturable(self) -> bool:
        """Whether a step of this model may be recorded into a CUDA graph: every part must say so."""
        return all(getattr(part, "capturable", False) for part in self.all_parts())

    # ---- weights ----------------------------------------------------------------------------------
    def named_parts(self):
        """(prefix, part) for every part that owns tensors."""
        yield self.spec.embedding.prefix, self.embedding
        for ls, block in zip(self.spec.layers, self.layers):
            yield ls.mixer_norm.prefix, block.mixer_norm
            yield ls.mixer.prefix, block.mixer
            yield ls.feed_forward_norm.prefix, block.feed_forward_norm
            yield ls.feed_forward.prefix, block.feed_forward
        yield self.spec.final_norm.prefix, self.final_norm
        yield self.spec.lm_head.prefix, self.lm_head
        for name, ps in self.spec.positions.items():
            yield ps.prefix, self.positions[name]

    def expected_tensors(self) -> dict:
        """full tensor name -> (part, name relative to the part, TensorSpec)."""
        out = {}
        for prefix, part in self.named_parts():
            for rel, tspec in part.tensor_specs().items():
                full = prefix + rel
                if full in out:
                    raise ValueError(f"two parts ask for tensor '{full}'")
                out[full] = (part, rel, tspec)
        return out

    def finish_loading(self) -> None:
        """Called once all tensors are in: the head may now borrow what it ties to from the embedding."""
        finish = getattr(self.lm_head, "finish", None)
        if finish is not None:
            finish(self.embedding)

    def weight_bytes(self) -> int:
        seen, total = set(), 0
        for _, part in self.named_parts():
            for t in getattr(part, "_tensors", {}).values():
                if t.data_ptr() not in seen:
                    seen.add(t.data_ptr())
                    total += t.numel() * t.element_size()
        return total

    # ---- one step -----------------------------------------------------------------------------------
    def forward(self, ctx) -> torch.Tensor:
        ctx.position_data = {name: pe.prepare(ctx) for name, pe in self.positions.items()}
        hidden = self.embedding.forward(ctx.tokens, ctx)
        stream = ResidualStream(hidden, None)
        for i, entry in enumerate(self.order):
            block = self.layers[entry.layer]
            following = self.layers[self.order[i + 1].layer] if i + 1 < len(self.order) else None
            stream.next_norm = following.first_norm() if following is not None else None
            cache = ctx.cache_view(entry.cache, entry.layer) if (entry.cache is not None or
                                                                block.mixer.state_spec() is not None) else None
            block.forward(stream, ctx, cache)
        if ctx.num_wanted == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=hidden.device)
        x = self.final_norm.add_norm(stream.hidden, stream.pending, ctx, rows=ctx.want_rows,
                                     upcoming=self.lm_head.first_weights())
        return self.lm_head.forward(x, ctx)
