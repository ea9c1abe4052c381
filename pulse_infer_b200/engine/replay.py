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

PAGE_SIZE = 16
TOKEN_ROUNDING = 64      # a request's token count is rounded up to this when sizing the pool
MAX_LIVE_REQUESTS = 8


def replay(model_dir: str, dtype: str, out_dir: str, max_tokens: int, lines, device="cuda:0", log=None) -> int:
    """Run the steps read from ``lines`` (an iterable of JSON strings); returns the number of steps."""
    os.makedirs(out_dir, exist_ok=True)
    pool_tokens = (max_tokens + TOKEN_ROUNDING - 1) // TOKEN_ROUNDING * TOKEN_ROUNDING
    runner = build_runner(model_dir, dtype=dtype, device=device, page_size=PAGE_SIZE, max_tokens=pool_tokens,
                          max_requests=MAX_LIVE_REQUESTS, max_tokens_per_request=pool_tokens)
    out = log or sys.stdout
    count = 0
    for line in lines:
        line = line.strip()
        if not line:
            continue
        obj = json.loads(line)
        step_id = obj["step"]
        segments = []
        for entry in obj.get("entries", []):
            rid = entry["id"]
            if not entry.get("tokens"):
                continue                      # an entry without tokens asks for nothing
            if not runner.cache.has(rid):
                runner.open(rid)
            segments.append(Segment(rid, [int(t) for t in entry["tokens"]], [int(w) for w in entry.get("want", [])]))
        if segments:
            logits = runner.step(segments)
            runner.check_device_errors()
            if logits.shape[0] > 0:
                arr = logits.detach().to("cpu", torch.float32).numpy().astype("<f4", copy=False)
                arr.tofile(os.path.join(out_dir, f"{step_id}.f32"))
        for rid in obj.get("end", []):
            if runner.cache.has(rid):
                runner.close(rid)
        print(f"done {step_id}", file=out, flush=True)
        count += 1
    return count
