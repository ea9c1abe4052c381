"""The generation loop: schedule -> one step -> sample -> finish and free, until no work is left.

Names follow ``include/pulse/scheduler/continuous_batch_engine.hpp:14-35``: ``add_request``,
``run_until_complete``, ``get_result``, ``get_request``, ``get_stats``; the loop is
``src/scheduler/continuous_batch_engine.cpp:80-112,140-257``.  Prompts are token ids (the reference
tokenizes text first, ``continuous_batch_engine.cpp:75-78``; text is outside this engine).  Logits are
asked for only at the last token of a request whose known tokens are all in; sampling runs on the
device.
"""
from __future__ import annotations

from ..sampling.params import SamplingParams
from .context import Segment
from .scheduler import ContinuousBatchScheduler, ScheduledBatch


class ContinuousBatchEngine:
    def __init__(self, runner, sampler, eos_token_ids=(), max_batch_size: int = 8, chunk_size: int = 256,
                 max_tokens_per_step: int | None = None, max_sequences: int | None = None):
        """``runner``: the step function (``open``/``close`` happen through its cache manager);
        ``sampler``: ``sample(logits, params, draw_index, history) -> token ids``."""
        self.runner = runner
        self.sampler = sampler
        self.eos_token_ids = tuple(eos_token_ids)
        cache = runner.cache
        self.scheduler = ContinuousBatchScheduler(cache, max_batch_size, max_sequences or cache.max_slots, chunk_size,
                                                  max_tokens_per_step)
        self.last_batch: ScheduledBatch | None = None

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
        return list(req.generated_tokens)

    def get_stats(self):
        return self.scheduler.get_stats()

    def abort(self, request_id: int) -> None:
        self.scheduler.abort(request_id)

    def has_work(self) -> bool:
        return self.scheduler.has_work()

    def step(self) -> list:
        """Plan and run one step.  Returns [(request id, sampled token)] for the requests that sampled."""
        batch = self.scheduler.schedule_next_batch()
        self.last_batch = batch
        if batch.empty():
            return []
        segments, sampling_reqs = [], []
        finished = []
        for req, n in batch.entries:
            tokens = req.get_next_chunk_tokens(n)
            all_in = req.num_computed_tokens + n == req.total_input_tokens()
            wants = all_in and req.can_generate_more()
            segments.append(Segment(req.request_id, tokens, [n - 1] if wants else []))
            if wants:
                sampling_reqs.append(req)
        logits = self.runner.step(segments)
        for req, n in batch.entries:
            req.add_computed_tokens(n)
        sampled = []
        if sampling_reqs:
            history = None
            if any(r.sampling.presence_penalty > 0.0 for r in sampling_reqs):
                history = [r.all_tokens() if r.sampling.presence_penalty > 0.0 else () for r in sampling_reqs]
            tokens = self.sampler.sample(logits, [r.sampling for r in sampling_reqs],
                                         [r.num_generated() for r in sampling_reqs], history)
            for req, tok in zip(sampling_reqs, tokens):
                keep_going = req.add_sampled_token(int(tok), self.eos_token_ids)
                sampled.append((req.request_id, int(tok)))
                if not keep_going:
                    finished.append(req.request_id)
        for req, n in batch.entries:
            # max_new_tokens == 0: finish right after the prompt without sampling (engine.cpp:197-206)
            if not req.is_finished() and not req.has_pending_input() and not req.can_generate_more():
                req.finish("length")
                finished.append(req.request_id)
        for rid in finished:
            self.runner.cache.close(rid)
        self.scheduler.update_after_step(batch, finished)
        return sampled

    def run_until_complete(self, on_step=None) -> None:
        while self.scheduler.has_work():
            out = self.step()
            if on_step is not None:
                on_step(self, out)
            if self.last_batch is not None and self.last_batch.empty() and not self.last_batch.failed \
                    and self.scheduler.has_work():
                raise RuntimeError("the scheduler planned nothing although work is left")
