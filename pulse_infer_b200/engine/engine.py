"""The generation loop: schedule -> one step -> sample -> finish and free, until no work is left.

Names follow ``include/pulse/scheduler/continuous_batch_engine.hpp:14-35``: ``add_request``,
``run_until_complete``, ``get_result``, ``get_request``, ``get_stats``; the loop is
``src/scheduler/continuous_batch_engine.cpp:80-112,140-257``.  Prompts are token ids (the reference
tokenizes text first, ``continuous_batch_engine.cpp:75-78``; text is outside this engine).  Logits are
asked for only at the last token of a request whose known tokens are all in; sampling runs on the
device.

With ``lookahead`` a step of single tokens stays in flight when ``step()`` returns: the ids it sampled are read
at the next call, after the next step has been launched with those ids taken straight from the device.  The
host's planning, packing and the read-back then run while the GPU works.  A request that ended with the token
read late (an EOS id) has run one token too far; that token is dropped.  ``step()`` returns the tokens of the
step before in that mode; results, finish reasons and the order of tokens per request are the same.
"""
from __future__ import annotations

from dataclasses import dataclass, field

from ..sampling.params import SamplingParams
from .context import Segment
from .scheduler import ContinuousBatchScheduler, ScheduledBatch


@dataclass
class _Launched:
    """A step that has been launched; its sampled ids may still be on the device."""
    batch: ScheduledBatch
    entries: list                                  # (request, tokens fed) that ran
    sampling_reqs: list = field(default_factory=list)
    tokens: object = None                          # device int32 [len(sampling_reqs)], or None
    host: object = None                            # pinned copy of ``tokens`` on its way to the host
    arrived: object = None                         # event behind that copy
    single_tokens: bool = False                    # every entry fed one token and sampled: the next step may chain on it


class ContinuousBatchEngine:
    def __init__(self, runner, sampler, eos_token_ids=(), max_batch_size: int = 8, chunk_size: int = 256,
                 max_tokens_per_step: int | None = None, max_sequences: int | None = None, lookahead: bool = False):
        """``runner``: the step function (``open``/``close`` happen through its cache manager);
        ``sampler``: ``sample(logits, params, draw_index, history) -> token ids``.
        ``lookahead`` needs ``sampler.sample_device`` and ``runner.step(..., tokens_from=)``."""
        self.runner = runner
        self.sampler = sampler
        self.lookahead = bool(lookahead)
        self._inflight: _Launched | None = None
        self._idle_step = False
        self._pinned: list = []                    # a few pinned buffers for sampled ids, used in turn
        self._pinned_turn = 0
        self.eos_token_ids = tuple(eos_token_ids)
        cache = runner.cache
        self.scheduler = ContinuousBatchScheduler(cache, max_batch_size, max_sequences or cache.max_slots, chunk_size,
                                                  max_tokens_per_step)
        self.last_batch: ScheduledBatch | None = None
        # called as logits_hook(requests that sample in this step, float32 logits [len(requests), vocab]) before sampling
        self.logits_hook = None

    def add_request(self, prompt_tokens, max_new_tokens: int, sampling: SamplingParams | None = None,
                    ignore_eos: bool = False) -> int:
        return self.scheduler.add_request(prompt_tokens, max_new_tokens, sampling, ignore_eos)

    def get_request(self, request_id: int):
        return self.scheduler.get_request(request_id)

    def get_result(self, request_id: int) -> list:
        """Generated token ids of a request (the EOS token, if one ended it, included)."""
        req = self.scheduler.get_request(request_id)
        if req is None:
            raise KeyError(f"unknown request {request_id}")
        return req.resolved_tokens()

    def get_stats(self):
        return self.scheduler.get_stats()

    def abort(self, request_id: int) -> None:
        self.scheduler.abort(request_id)

    def has_work(self) -> bool:
        return self.scheduler.has_work() or self._inflight is not None

    def step(self) -> list:
        """Plan and run one step.  Returns [(request id, sampled token)] for the requests that sampled (with
        ``lookahead``: of the step that was in flight)."""
        prev, self._inflight = self._inflight, None
        batch = self.scheduler.schedule_next_batch()
        self.last_batch = batch
        self._idle_step = batch.empty() and not batch.failed and prev is None
        out = []
        if batch.empty():
            return self._collect(prev) if prev is not None else out
        if prev is None:
            rec = self._launch(batch)
        elif not any(req.unresolved for req, _ in batch.entries):
            rec = self._launch(batch)                  # nothing here feeds on what is still on the device
            out = self._collect(prev)
        elif self._chains_on(batch, prev):
            rec = self._launch(batch, tokens_from=prev.tokens)     # the GPU goes on; the host reads the step before
            out = self._collect(prev)
        else:
            out = self._collect(prev)                  # the ids are needed on the host first
            rec = self._launch(batch)
        if rec is not None:
            if self.lookahead and rec.single_tokens:
                self._inflight = rec
            else:
                out = out + self._collect(rec)
        return out

    def _chains_on(self, batch: ScheduledBatch, prev: _Launched) -> bool:
        """The planned step is one token for each request that sampled in ``prev``, in the same order."""
        if prev.tokens is None or len(batch.entries) != len(prev.sampling_reqs):
            return False
        return all(n == 1 and req is p and req.unresolved == 1
                   and req.num_computed_tokens + 1 == req.total_input_tokens()      # the id in flight is what it feeds
                   for (req, n), p in zip(batch.entries, prev.sampling_reqs))

    def _launch(self, batch: ScheduledBatch, tokens_from=None) -> _Launched | None:
        entries = [(req, n) for req, n in batch.entries if not req.is_finished()]     # ended by the read-back just before
        segments, sampling_reqs = [], []
        for req, n in entries:
            tokens = req.get_next_chunk_tokens(n)
            all_in = req.num_computed_tokens + n == req.total_input_tokens()
            wants = all_in and req.can_generate_more()
            segments.append(Segment(req.request_id, tokens, [n - 1] if wants else []))
            if wants:
                sampling_reqs.append(req)
        rec = _Launched(batch, entries)
        if not segments:
            return rec
        if tokens_from is not None:
            logits = self.runner.step(segments, tokens_from=tokens_from)
        else:
            logits = self.runner.step(segments)
        for req, n in entries:
            req.add_computed_tokens(n)
        if sampling_reqs:
            if self.logits_hook is not None:
                self.logits_hook(sampling_reqs, logits)
            history = None
            if any(r.sampling.presence_penalty > 0.0 for r in sampling_reqs):
                history = [r.all_tokens() if r.sampling.presence_penalty > 0.0 else () for r in sampling_reqs]
            params = [r.sampling for r in sampling_reqs]
            draws = [r.num_generated() for r in sampling_reqs]
            rec.sampling_reqs = sampling_reqs
            if self.lookahead:
                rec.tokens = self.sampler.sample_device(logits, params, draws, history)
                self._start_read_back(rec)
                # the next step may chain on this one if it is the steady state of decoding: one token each, all
                # sampling, nothing that looks at earlier tokens on the host, and a step that takes device tokens
                rec.single_tokens = (len(sampling_reqs) == len(entries) and all(n == 1 for _, n in entries)
                                     and not any(p.edits_logits for p in params)
                                     and self.runner.takes_device_tokens(segments))
            else:
                rec.tokens = self.sampler.sample(logits, params, draws, history)
            for r in sampling_reqs:
                r.add_pending_token()
        return rec

    def _start_read_back(self, rec: _Launched) -> None:
        """Queue the copy of the sampled ids to pinned host memory right behind the sampling kernel - before the next
        step is launched, so that waiting for it does not wait for that step."""
        tokens = rec.tokens
        if not getattr(tokens, "is_cuda", False):
            return
        import torch
        n = tokens.numel()
        if not self._pinned or self._pinned[0].numel() < n:
            self._pinned = [torch.empty(max(n, 64), dtype=torch.int32).pin_memory() for _ in range(4)]
        self._pinned_turn = (self._pinned_turn + 1) % len(self._pinned)
        rec.host = self._pinned[self._pinned_turn][:n]
        rec.host.copy_(tokens.reshape(-1), non_blocking=True)
        rec.arrived = torch.cuda.Event()
        rec.arrived.record()

    def _collect(self, rec: _Launched | None) -> list:
        """Read the ids a launched step sampled, append them, finish and free."""
        if rec is None:
            return []
        sampled, finished = [], []
        if rec.sampling_reqs:
            if rec.arrived is not None:
                rec.arrived.synchronize()
                tokens = rec.host.tolist()
            else:
                tokens = rec.tokens if isinstance(rec.tokens, list) else rec.tokens.tolist()
            for req, tok in zip(rec.sampling_reqs, tokens):
                if req.is_finished():                  # ended (or was aborted) while this step was in flight
                    req.drop_pending_tokens()
                    continue
                keep_going = req.resolve_pending_token(int(tok), self.eos_token_ids)
                sampled.append((req.request_id, int(tok)))
                if not keep_going:
                    finished.append(req.request_id)
        for req, n in rec.entries:
            # max_new_tokens == 0: finish right after the prompt without sampling (engine.cpp:197-206)
            if (not req.is_finished() and not req.unresolved and not req.has_pending_input()
                    and not req.can_generate_more()):
                req.finish("length")
                finished.append(req.request_id)
        for rid in finished:
            # a request that was preempted while its last id was still on its way holds no slot any more (the
            # scheduler gave its pages back and put it in the waiting queue; update_after_step takes it out there)
            if self.runner.cache.has(rid):
                self.runner.cache.close(rid)
        self.scheduler.update_after_step(rec.batch, finished)
        return sampled

    def run_until_complete(self, on_step=None) -> None:
        while self.has_work():
            out = self.step()
            if on_step is not None:
                on_step(self, out)
            if self._idle_step and self.scheduler.has_work():
                raise RuntimeError("the scheduler planned nothing although work is left")
