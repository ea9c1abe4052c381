"""The Python entry point: ``Engine`` wraps configuration, weights, cache, step function, scheduler
and sampler behind the calls the reference's batching engine offers
(``include/pulse/scheduler/continuous_batch_engine.hpp:14-35``): ``add_request``,
``run_until_complete``, ``get_result``, ``get_request``, ``get_stats`` - plus ``generate`` for the common
case.  Prompts and results are lists of token ids.

    from pulse_infer_b200 import Engine
    engine = Engine("/path/to/model", dtype="bfloat16", max_batch_size=8)
    outputs = engine.generate([[1, 2, 3], [4, 5]], max_new_tokens=32)
"""
from __future__ import annotations

from .engine.builder import build_runner
from .engine.engine import ContinuousBatchEngine
from .sampling import Sampler, SamplingParams


class Engine:
    def __init__(self, model: str | None = None, *, config=None, seed: int | None = None, dtype: str = "bfloat16",
                 device: str = "cuda:0", page_size: int = 16, num_pages: int | None = None,
                 max_tokens: int | None = None, max_batch_size: int = 8, chunk_size: int = 1024,
                 max_tokens_per_step: int | None = None, max_tokens_per_request: int | None = None,
                 use_cuda_graphs: bool = True, attention_impl: str = "auto", rope_pairing: str | None = None,
                 lookahead: bool | None = None, kv_bytes: int | None = None):
        """``model``: folder with config.json and safetensors; or ``config`` + ``seed`` for random weights.
        The page pool is ``num_pages`` pages of ``page_size`` tokens, or what fits in ``kv_bytes`` bytes, or enough
        for ``max_tokens`` tokens
        (default: ``max_batch_size`` requests of the model's longest context, capped at 1M tokens).
        ``chunk_size`` (longest prompt portion of one request in one step) defaults to 1,024 and ``max_tokens_per_step``
        to 2,048 (or ``chunk_size`` if that is larger): on a B200 a step of 128 or 256 prompt tokens costs as much as
        one of 512 (the weights are read either way), and 1,024-token portions reach the prompt throughput of whole
        prompts, while a step stays short enough for the decoding requests that ride along.
        ``lookahead`` (default: on with CUDA graphs): a decode step stays in flight when ``step()`` returns and its
        tokens are read while the next one runs; ``step()`` then returns the tokens of the step before."""
        spec_options = {} if rope_pairing is None else {"rope_pairing": rope_pairing}
        self.runner = build_runner(model, config=config, seed=seed, dtype=dtype, device=device, page_size=page_size,
                                   num_pages=num_pages, max_tokens=max_tokens, max_requests=max(max_batch_size, 1),
                                   max_tokens_per_request=max_tokens_per_request,
                                   max_tokens_per_step=None, attention_impl=attention_impl,
                                   use_cuda_graphs=use_cuda_graphs, kv_bytes=kv_bytes, **spec_options)
        self.config = self.runner.config
        self.sampler = Sampler(self.runner.runtime.device)
        self.engine = ContinuousBatchEngine(self.runner, self.sampler, getattr(self.config, "eos_token_ids", ()),
                                            max_batch_size=max_batch_size, chunk_size=chunk_size,
                                            max_tokens_per_step=max_tokens_per_step or max(2048, chunk_size),
                                            lookahead=use_cuda_graphs if lookahead is None else lookahead)

    # ---- the reference engine's calls ------------------------------------------------------------------
    def add_request(self, prompt_tokens, max_new_tokens: int = 32, *, temperature: float = 0.0, top_k: int = 0,
                    top_p: float = 0.0, presence_penalty: float = 0.0, banned_tokens=(), seed: int = 0,
                    ignore_eos: bool = False) -> int:
        params = SamplingParams(temperature=temperature, top_k=top_k, top_p=top_p, presence_penalty=presence_penalty,
                                banned_tokens=tuple(banned_tokens), seed=seed)
        return self.engine.add_request(list(prompt_tokens), max_new_tokens, params, ignore_eos)

    def step(self) -> list:
        return self.engine.step()

    def has_work(self) -> bool:
        return self.engine.has_work()

    def run_until_complete(self, on_step=None) -> None:
        self.engine.run_until_complete(on_step)

    def get_result(self, request_id: int) -> list:
        return self.engine.get_result(request_id)

    def get_request(self, request_id: int):
        return self.engine.get_request(request_id)

    def get_stats(self):
        return self.engine.get_stats()

    def abort(self, request_id: int) -> None:
        self.engine.abort(request_id)

    # ---- convenience ---------------------------------------------------------------------------------------
    def run(self) -> dict:
        """Run until no request is left; returns {request id: generated ids} of every request that has finished."""
        self.run_until_complete()
        return {rid: req.resolved_tokens() for rid, req in self.engine.scheduler.request_map.items() if req.is_finished()}

    def replay(self, trace) -> dict:
        """Feed given token ids through this engine's own step function, step by step, sampling nothing: ``trace`` is
        a list of steps ``{"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}``
        (dicts or JSON strings, as ``bin/trace_run`` reads them); returns {step: float32 logits [wanted, vocab]} for
        the steps in which something was wanted.  The engine must be idle, and the trace's ids its own."""
        from .engine.replay import replay_steps
        if self.has_work():
            raise RuntimeError("replay needs an engine without requests in flight")
        return {step_id: logits for step_id, _, logits in replay_steps(self.runner, trace) if logits is not None}

    def warm_up(self, batch_sizes=None) -> int:
        """Records the decode step of every batch size up to ``max_batch_size`` (or of ``batch_sizes``) before traffic
        arrives, as a server does at start-up.  Recording a step takes tens of milliseconds the first time a batch size
        occurs; a short run that meets many batch sizes (requests finishing one after the other) otherwise spends a
        tenth of its time on it.  Each size is recorded by one step of that many one-token requests.  Returns the
        number of steps recorded; 0 without CUDA graphs.  (The reference has no counterpart: it launches every kernel
        eagerly.)"""
        graphs = self.runner.graphs
        if graphs is None:
            return 0
        before = graphs.recordings
        limit = min(self.engine.scheduler.max_batch_size, graphs.max_graphs)
        sizes = sorted({int(b) for b in (batch_sizes or range(1, limit + 1)) if 1 <= int(b) <= limit}, reverse=True)
        for b in sizes:
            for _ in range(b):
                self.add_request([0], 1, ignore_eos=True)
            self.run_until_complete()
        return graphs.recordings - before

    def generate(self, prompts, max_new_tokens: int = 32, **sampling) -> list:
        """Generate for a list of prompts (each a list of token ids); returns the generated ids of each."""
        ids = [self.add_request(p, max_new_tokens, **sampling) for p in prompts]
        self.run_until_complete()
        return [self.get_result(i) for i in ids]
