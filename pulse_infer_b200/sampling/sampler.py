"""Choosing the next token of every request of a step, on the device.

Greedy rows use the argmax kernel; rows with a temperature use the sampling kernel (temperature,
top-k, top-p; a counter-based uniform draw keyed by the request's seed and the index of the draw, so
a request's tokens do not depend on what else is in the batch or on being recomputed after a
preemption).  Presence penalty and banned ids edit single logits first.

Reference parity: ``src/scheduler/continuous_batch_engine.cpp:237,259-305`` (greedy on the last row of
each request) and ``demo/qwen3_infer.cpp:229-423`` (the sampler of the single-stream demo).
"""
from __future__ import annotations

import torch

from .. import ops
from .params import SamplingParams


class Sampler:
    def __init__(self, device):
        self.device = torch.device(device)

    def sample(self, logits: torch.Tensor, params: list, draw_index: list, history: list | None = None) -> list:
        """logits float32 [n, V]; params[i] SamplingParams; draw_index[i] how many tokens request i has
        drawn so far; history[i] the tokens a presence penalty looks at.  Returns n token ids."""
        out = self.sample_device(logits, params, draw_index, history)
        return [] if out is None else out.tolist()

    def sample_device(self, logits: torch.Tensor, params: list, draw_index: list, history: list | None = None):
        """The same, but the token ids stay on the device (int32 [n], or None for no rows): the caller reads them
        when it needs them, and the next step can take them as its input without a round trip."""
        n = logits.shape[0]
        if n == 0:
            return None
        if any(p.edits_logits for p in params):
            logits = logits.clone()
            rows, toks, vals_add, rows_set, toks_set = [], [], [], [], []
            for i, p in enumerate(params):
                if p.presence_penalty > 0.0 and history is not None:
                    for t in set(history[i]):
                        rows.append(i); toks.append(t); vals_add.append(-p.presence_penalty)
                for t in set(p.banned_tokens):
                    rows_set.append(i); toks_set.append(t)
            mk = lambda v, dt: torch.tensor(v, dtype=dt, device=self.device)  # noqa: E731
            if rows:
                ops.logit_edit(logits, mk(rows, torch.int32), mk(toks, torch.int32), mk(vals_add, torch.float32), False)
            if rows_set:
                ops.logit_edit(logits, mk(rows_set, torch.int32), mk(toks_set, torch.int32),
                               mk([float("-inf")] * len(rows_set), torch.float32), True)
        if all(p.greedy for p in params):
            return ops.argmax(logits)
        mk = lambda v, dt: torch.tensor(v, dtype=dt, device=self.device)  # noqa: E731
        out = ops.sample(
            logits,
            mk([0.0 if p.greedy else p.temperature for p in params], torch.float32),
            mk([p.top_k for p in params], torch.int32),
            mk([p.top_p for p in params], torch.float32),
            mk([_as_i64(p.seed) for p in params], torch.int64),
            mk(list(draw_index), torch.int64))
        return out


def _as_i64(v: int) -> int:
    v &= (1 << 64) - 1
    return v - (1 << 64) if v >= (1 << 63) else v
