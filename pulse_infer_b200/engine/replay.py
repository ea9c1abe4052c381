"""Trace replay: feed given token ids through the step function, step by step, and write logits.

Nothing is sampled and nothing is scheduled; the trace says exactly which tokens of which request go
into which step.  It drives the same model, step function, cache manager and kernels as generation.
Input: one JSON object per line,
``{"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": ["b"]}``.
For a step in which something is wanted, ``<out>/<step>.f32`` holds the logits at the wanted places
(order of the entries and of ``want``) as little-endian float32 ``[wanted, vocab]``.
The reference has nothing comparable.
"""
from __future__ import annotations

import json
import os
import sys

import numpy as np
import torch

from .builder import build_runner
from .context import Segment

PAGE_SIZE = 16           # default page size in tokens
TOKEN_ROUNDING = 64      # a request's token count is rounded up to this when sizing the pool
MAX_LIVE_REQUESTS = 8    # default number of request slots


def replay_steps(runner, steps):
    """The steps of a trace through a runner's step function, one after the other: yields (step id, the step's
    segments, float32 logits [wanted, vocab] as a numpy array or None when nothing was wanted).  ``steps``: JSON
    strings or dicts of the form shown above.  Requests are opened at their first tokens and closed where ``end``
    names them."""
    for step in steps:
        if isinstance(step, str):
            step = step.strip()
            if not step:
                continue
            step = json.loads(step)
        step_id = step["step"]
        segments = []
        for entry in step.get("entries", []):
            rid = entry["id"]
            if not entry.get("tokens"):
                continue                      # an entry without tokens asks for nothing
            if not runner.cache.has(rid):
                runner.open(rid)
            segments.append(Segment(rid, [int(t) for t in entry["tokens"]], [int(w) for w in entry.get("want", [])]))
        arr = None
        if segments:
            logits = runner.step(segments)
            runner.check_device_errors()
            if logits.shape[0] > 0:
                arr = logits.detach().to("cpu", torch.float32).numpy()
        for rid in step.get("end", []):
            if runner.cache.has(rid):
                runner.close(rid)
        yield step_id, segments, arr


def replay(model_dir: str, dtype: str, out_dir: str, max_tokens: int | None, lines, device="cuda:0", log=None,
           page_size: int = PAGE_SIZE, num_pages: int | None = None, max_requests: int = MAX_LIVE_REQUESTS) -> int:
    """Run the steps read from ``lines`` (an iterable of JSON strings); returns the number of steps.
    The pool holds ``num_pages`` pages of ``page_size`` tokens, or enough for ``max_tokens`` tokens (each request's
    count rounded up to a multiple of 64 or of the page size, whichever is larger).  Beside the ``.f32`` files,
    ``index.json`` lists for every row written: step, request, position of the token in its request, row."""
    os.makedirs(out_dir, exist_ok=True)
    if page_size <= 0:
        raise ValueError("page_size must be positive")
    if num_pages is None:
        if max_tokens is None:
            raise ValueError("give max_tokens or num_pages")
        rounding = max(TOKEN_ROUNDING, page_size)
        pool_tokens = (max_tokens + rounding - 1) // rounding * rounding
        num_pages = (pool_tokens + page_size - 1) // page_size
    pool_tokens = num_pages * page_size
    runner = build_runner(model_dir, dtype=dtype, device=device, page_size=page_size, num_pages=num_pages,
                          max_requests=max_requests, max_tokens_per_request=pool_tokens)
    out = log or sys.stdout
    count = 0
    index = []
    for step_id, segments, logits in replay_steps(runner, lines):
        if logits is not None:
            logits.astype("<f4", copy=False).tofile(os.path.join(out_dir, f"{step_id}.f32"))
            row = 0
            for seg in segments:
                for w in seg.want:
                    index.append({"step": step_id, "request": seg.request_id, "position": seg.start + w, "row": row})
                    row += 1
        print(f"done {step_id}", file=out, flush=True)
        count += 1
    with open(os.path.join(out_dir, "index.json"), "w", encoding="utf-8") as fh:
        json.dump({"page_size": page_size, "num_pages": num_pages, "dtype": dtype, "rows": index}, fh)
    return count
