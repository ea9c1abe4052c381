"""The step function: ONE entry point that runs a batch of (request, its next tokens) through the
model from the cache and returns the logits at the wanted places.

A batch may mix portions of prompts of any length with single decoded tokens.  Only the tokens given
are computed; everything earlier comes from the pages that earlier steps filled.  Pages are reserved
before the model runs (so a step either has all its pages or does not start) and lengths are
committed after it.

Reference parity: ``src/model/qwen3/model.cpp:1179-1374`` (``forward_batched``) - same inputs in spirit
(tokens, absolute positions, sequence ids), but the reference allocates pages while walking the tokens
(``model.cpp:1204-1250``), reallocates its workspaces when the token count changes (``model.cpp:467-587``)
and returns logits for every row.
"""
from __future__ import annotations

import torch

from ..cache import CacheManager
from .context import Segment, StepContext


class StepError(ValueError):
    pass


class ModelRunner:
    def __init__(self, model, cache_manager: CacheManager, runtime, max_tokens_per_step: int | None = None,
                 use_cuda_graphs: bool = False):
        self.model = model
        self.cache = cache_manager
        self.runtime = runtime
        self.max_tokens_per_step = max_tokens_per_step
        self.vocab_size = model.spec.vocab_size
        self.max_position = model.spec.max_position
        self._last_ctx: StepContext | None = None
        self.graphs = None
        if use_cuda_graphs:
            from .graphs import DecodeGraphs
            self.graphs = DecodeGraphs(self)

    # ---- requests ------------------------------------------------------------------------------------
    def open(self, request_id) -> int:
        return self.cache.open(request_id)

    def close(self, request_id) -> None:
        self.cache.close(request_id)

    # ---- the step ---------------------------------------------------------------------------------------
    def prepare(self, segments: list) -> None:
        """Validate the batch, resolve slots and start positions, reserve pages."""
        if not segments:
            raise StepError("a step needs at least one segment")
        seen = set()
        total = 0
        for s in segments:
            if s.request_id in seen:
                raise StepError(f"request '{s.request_id}' appears twice in one step")
            seen.add(s.request_id)
            n = len(s.tokens)
            if n == 0:
                raise StepError(f"request '{s.request_id}' brings no tokens")
            total += n
            lowest, highest = (s.tokens[0], s.tokens[0]) if n == 1 else (min(s.tokens), max(s.tokens))
            if lowest < 0 or highest >= self.vocab_size:
                bad = lowest if lowest < 0 else highest
                raise StepError(f"request '{s.request_id}': token id {bad} is outside the vocabulary "
                                f"[0, {self.vocab_size})")
            s.slot = self.cache.slot(s.request_id)
            s.start = self.cache.length(s.request_id)
            if s.start + n > self.max_position:
                raise StepError(f"request '{s.request_id}' would reach position {s.start + n - 1}, beyond "
                                f"max_position_embeddings = {self.max_position}")   # model.cpp:1209-1211
        if self.max_tokens_per_step is not None and total > self.max_tokens_per_step:
            raise StepError(f"{total} tokens in one step, the limit is {self.max_tokens_per_step}")
        for s in segments:
            self.cache.reserve(s.request_id, s.start + len(s.tokens))

    def takes_device_tokens(self, segments: list) -> bool:
        """Whether ``step(segments, tokens_from=...)`` is possible: a captured step of single tokens."""
        return self.graphs is not None and self.graphs.eligible(segments)

    def step(self, segments: list, tokens_from: torch.Tensor | None = None) -> torch.Tensor:
        """segments: list of ``Segment(request_id, tokens, want)``.  Returns float32 logits
        [number of wanted places, vocab] in the order of the segments and of their ``want`` lists.
        ``tokens_from`` (int32 on the device, one id per segment, captured steps only): the input tokens are taken
        from there instead of from the segments - the ids the previous step sampled, not yet read by the host."""
        self.prepare(segments)
        self.cache.sync_tables()
        if tokens_from is not None and not self.takes_device_tokens(segments):
            raise StepError("tokens can come from the device only in a captured step of single tokens")
        if self.graphs is not None and self.graphs.eligible(segments):
            logits = self.graphs.run(segments, tokens_from)      # valid until the next captured step runs
            ctx = None
        else:
            ctx = StepContext.build(segments, self.runtime, self.cache)
            logits = self.model.forward(ctx)
        for s in segments:
            self.cache.commit(s.request_id, s.start + len(s.tokens))
        if ctx is not None:
            self._last_ctx = ctx
        return logits

    def check_device_errors(self) -> None:
        """Raise if a kernel of the last step met a token without a page (costs a device sync)."""
        if self._last_ctx is not None and self._last_ctx.error_count is not None:
            bad = int(self._last_ctx.error_count.item())
            if bad:
                raise StepError(f"{bad} key/value rows had no page to go to: block table and batch disagree")
        if self.runtime.mode == "bfloat16":
            from .. import ops
            status = ops.gemm_tcgen05_status()
            if status:
                raise StepError(f"a wait inside the tcgen05 product ran out (status {status:#x})")
            status = ops.attention_tcgen05_loaded_status()
            if status:
                raise StepError(f"a wait inside the tcgen05 attention kernel ran out (status {status:#x})")
