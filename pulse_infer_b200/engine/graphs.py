"""Decode steps as CUDA graphs.

A step that holds only single decoded tokens launches a few hundred small kernels; at batch 1 their
launch cost exceeds their run time.  Such a step is captured once per (number of requests, and for layers
whose decode attention cuts keys into ranges a bound on their number) and replayed: the metadata buffer, the block tables and the output live at fixed
addresses and are refilled in place before each replay.  The captured work is exactly what the eager
step runs (same model code, same kernels).  The reference launches everything eagerly on the null
stream (``src/ops/rope.cpp:231``, ``src/ops/matmul.cpp:115``).
"""
from __future__ import annotations

import gc
import time

import torch

from .. import ops
from .context import StepContext


def _pow2_at_least(n: int) -> int:
    p = 1
    while p < n:
        p *= 2
    return p


class DecodeGraph:
    def __init__(self, runner, num_requests: int, split_keys: tuple, splits_bound: int, pool=None, logits_out=None):
        self.runner = runner
        self.pool = pool
        self.num_requests = num_requests
        self.splits_bound = splits_bound
        device = runner.runtime.device
        self.layout = StepContext.layout(num_requests, num_requests, num_requests)
        total = self.layout["_total"][1]
        # two pinned staging buffers used in turn: a buffer is not rewritten before its copy has run
        self.hosts = [torch.zeros(total, dtype=torch.int32).pin_memory() for _ in range(2)]
        self.copied = [None, None]
        self.turn = 0
        self.ctx = StepContext(runner.runtime, runner.cache)
        self.ctx.buffer = torch.zeros(total, dtype=torch.int32, device=device)
        self.ctx.error_count = torch.zeros(1, dtype=torch.int32, device=device)
        self.ctx.splits_bound = splits_bound
        self.ctx.split_keys = dict(split_keys)
        self.ctx.logits_out = logits_out
        self.graph: torch.cuda.CUDAGraph | None = None
        self.logits: torch.Tensor | None = None

    def _refill(self, segments) -> None:
        buf, lay, (T, R, W) = StepContext.pack(segments)
        assert lay == self.layout
        i = self.turn
        self.turn ^= 1
        if self.copied[i] is not None:
            self.copied[i].synchronize()
        self.hosts[i].numpy()[:] = buf
        self.ctx.buffer.copy_(self.hosts[i], non_blocking=True)
        self.copied[i] = torch.cuda.Event()
        self.copied[i].record()
        self.ctx._bind(segments, lay, T, R, W)

    def run(self, segments, tokens_from=None) -> torch.Tensor:
        self._refill(segments)
        if tokens_from is not None:      # ids sampled by the step before, still on the device
            if tokens_from.dtype != torch.int32 or tokens_from.numel() != self.num_requests:
                raise ValueError("tokens_from must hold one int32 id per request of the step")
            self.ctx.tokens.copy_(tokens_from.reshape(-1))
        if self.graph is None:
            t0 = time.perf_counter()
            model = self.runner.model
            # Once eagerly (library initialisation, kernel attributes), then capture the same work.  The eager run and
            # the first replay both compute this step: page writes are idempotent, and fixed-size per-request state
            # is put back to what it was, so that the replay finds the step's true input there.
            states = self.runner.cache.state
            kept = {layer: t.clone() for layer, t in states.items() if t is not None}
            model.forward(self.ctx)
            for layer, t in kept.items():
                states[layer].copy_(t)
            del kept
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            before = ops.kernels.LAUNCHES
            # No garbage collection while the stream is capturing: collecting an old CUDAGraph object (of an engine
            # that is no longer used) destroys its graph, which is not permitted during a capture and invalidates it.
            collecting = gc.isenabled()
            gc.disable()
            try:
                with torch.cuda.graph(graph, pool=self.pool):
                    self.logits = model.forward(self.ctx)
            finally:
                if collecting:
                    gc.enable()
            self.launches_per_replay = ops.kernels.LAUNCHES - before
            self.graph = graph
            self.record_seconds = time.perf_counter() - t0
        self.graph.replay()
        ops.kernels.count_launches(self.launches_per_replay)
        return self.logits


class DecodeGraphs:
    """The captured decode steps of one runner, made on demand, a bounded number kept."""

    def __init__(self, runner, max_graphs: int = 96):
        self.runner = runner
        self.max_graphs = max_graphs
        self.graphs: dict = {}
        self.recordings = 0            # steps recorded so far, and the host time that took
        self.record_seconds = 0.0
        # Recorded steps run one at a time, so they share one memory pool for what they allocate while being recorded
        # and one home for their logits (valid until the next recorded step runs): the memory of the recordings is
        # that of the largest one, not their sum (a [batch, vocabulary] float32 tensor for every batch size otherwise).
        self.pool = None
        self.logits_out = None

    def eligible(self, segments) -> bool:
        """A step of single tokens, each wanting its logits, of a model whose parts all allow recording
        (``parts.base.Part.capturable``); everything else is launched kernel by kernel."""
        if not getattr(self.runner.model, "capturable", False) or len(segments) > ops.DECODE_MAX_SEGMENTS:
            return False
        return all(len(s.tokens) == 1 and list(s.want) == [0] for s in segments)

    def run(self, segments, tokens_from=None) -> torch.Tensor:
        # kinds of layers whose decode attention works on key ranges (parts that do not say are taken to)
        page_size, act_dtype = self.runner.cache.page_size, self.runner.runtime.act_dtype
        specs = set()
        for part in self.runner.model.all_parts():
            spec_of = getattr(part, "cache_spec", None)
            cs = spec_of() if spec_of is not None else None
            uses = getattr(part, "uses_key_ranges", None)
            if cs is not None and (uses is None or uses(page_size, act_dtype)):
                specs.add(cs)
        starts = [s.start for s in segments]
        pos_max = max(starts)
        # keys per range for every kind of layer (kv heads, head size), and one bound on the ranges for the whole
        # step: the widest request of the widest kind
        split_keys = {}
        for cs in specs:
            split_keys[(cs.num_kv_heads, cs.head_dim)] = ops.choose_split_keys(len(segments), cs.num_kv_heads, pos_max,
                                                                               cs.head_dim)
        need = max((ops.attention_splits_bound(starts, cs.window, split_keys[(cs.num_kv_heads, cs.head_dim)])
                    for cs in specs), default=1)
        key = (len(segments), tuple(sorted(split_keys.items())), _pow2_at_least(need))
        g = self.graphs.get(key)
        if g is None:
            if len(self.graphs) >= self.max_graphs:
                self.graphs.pop(next(iter(self.graphs)))
            if self.pool is None:
                self.pool = torch.cuda.graph_pool_handle()
                self.logits_out = torch.empty((self.runner.cache.max_slots, self.runner.model.spec.vocab_size),
                                              dtype=torch.float32, device=self.runner.runtime.device)
            g = DecodeGraph(self.runner, *key, pool=self.pool, logits_out=self.logits_out)
            self.graphs[key] = g
        fresh = g.graph is None
        logits = g.run(segments, tokens_from)
        if fresh:
            self.recordings += 1
            self.record_seconds += g.record_seconds
        return logits
