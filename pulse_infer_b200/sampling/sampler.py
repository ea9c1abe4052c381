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
    """Sampling options live in small device tables, one entry per distinct set of options, written once when a
    request with new options first samples.  A step then ships only one int64 pair per row - (table entry, draw
    counter) - in a single copy from pinned memory."""

    def __init__(self, device, table_entries: int = 1024, max_rows: int = 256):
        self.device = torch.device(device)
        self.table_entries = table_entries
        self._entry_of: dict = {}             # (temperature, top_k, top_p, seed) -> entry, in order of last use
        self._tables = None
        self._staging: list = []              # pinned buffers for the per-step pairs, used in turn
        self._copied: list = []
        self._turn = 0
        self._max_rows = max_rows

    # ---- option tables -------------------------------------------------------------------------------------
    def _ensure_tables(self) -> None:
        if self._tables is None:
            n, dev = self.table_entries, self.device
            self._tables = (torch.zeros(n, dtype=torch.float32, device=dev), torch.zeros(n, dtype=torch.int32, device=dev),
                            torch.zeros(n, dtype=torch.float32, device=dev), torch.zeros(n, dtype=torch.int64, device=dev))

    def _entry(self, p: SamplingParams) -> int:
        key = (0.0 if p.greedy else float(p.temperature), int(p.top_k), float(p.top_p), _as_i64(p.seed))
        entry = self._entry_of.pop(key, None)
        if entry is None:
            if len(self._entry_of) < self.table_entries:
                entry = len(self._entry_of)
            else:                              # the table is full: the entry unused for longest is overwritten
                oldest = next(iter(self._entry_of))
                entry = self._entry_of.pop(oldest)
            temperature, top_k, top_p, seeds = self._tables
            temperature[entry], top_k[entry], top_p[entry], seeds[entry] = key
        self._entry_of[key] = entry            # most recently used last
        return entry

    def _pairs_to_device(self, pairs: list) -> torch.Tensor:
        n = len(pairs)
        if not self._staging or self._staging[0].shape[0] < n:
            self._max_rows = max(self._max_rows, n)
            self._staging = [torch.empty((self._max_rows, 2), dtype=torch.int64).pin_memory() for _ in range(4)]
            self._copied = [None] * 4
        i = self._turn
        self._turn = (self._turn + 1) % len(self._staging)
        if self._copied[i] is not None:
            self._copied[i].synchronize()      # the copy that last used this buffer has run
        host = self._staging[i][:n]
        host.copy_(torch.tensor(pairs, dtype=torch.int64))
        dev = host.to(self.device, non_blocking=True)
        self._copied[i] = torch.cuda.Event()
        self._copied[i].record()
        return dev

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
        self._ensure_tables()
        if n > self.table_entries:
            raise ValueError(f"{n} rows in one step, the sampler's option tables hold {self.table_entries} entries")
        pairs = [[self._entry(p), int(c)] for p, c in zip(params, draw_index)]
        temperature, top_k, top_p, seeds = self._tables
        return ops.sample_entries(logits, temperature, top_k, top_p, seeds, self._pairs_to_device(pairs))


def _as_i64(v: int) -> int:
    v &= (1 << 64) - 1
    return v - (1 << 64) if v >= (1 << 63) else v
