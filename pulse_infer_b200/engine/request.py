"""One generation request and its life: WAITING -> RUNNING -> FINISHED.

Names and meanings follow ``include/pulse/scheduler/inference_request.hpp:15-199``: prompt tokens,
generated tokens, ``num_computed_tokens`` (how much of prompt + generated already sits in the cache),
chunk cutting (``get_next_chunk_size``: a prompt portion while prefilling, else the one pending
token), finishing on an EOS id, on token -1 or at ``max_new_tokens`` with the EOS token kept in the
output (``inference_request.hpp:130-143``).  Added: sampling options, a finish reason, and preemption
(the request goes back to WAITING and will recompute prompt + generated tokens).
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from enum import Enum

from ..sampling.params import SamplingParams


class RequestState(Enum):
    WAITING = "waiting"
    RUNNING = "running"
    FINISHED = "finished"


@dataclass(eq=False)        # a request is itself, not its field values: the scheduler's lists compare by identity
class InferenceRequest:
    request_id: int
    prompt_tokens: list
    max_new_tokens: int
    sampling: SamplingParams = field(default_factory=SamplingParams)
    ignore_eos: bool = False
    generated_tokens: list = field(default_factory=list)
    state: RequestState = RequestState.WAITING
    num_computed_tokens: int = 0
    finish_reason: str | None = None
    num_preemptions: int = 0
    unresolved: int = 0          # trailing entries of generated_tokens that were sampled but not read back yet
    arrival_time: float = field(default_factory=time.monotonic)
    start_time: float | None = None
    finish_time: float | None = None

    # ---- inference_request.hpp:57-87 ------------------------------------------------------------------
    def prompt_len(self) -> int:
        return len(self.prompt_tokens)

    def num_generated(self) -> int:
        return len(self.generated_tokens)

    def total_input_tokens(self) -> int:
        return self.prompt_len() + self.num_generated()

    def is_finished(self) -> bool:
        return self.state == RequestState.FINISHED

    def is_prefill(self) -> bool:
        """Feeding tokens that are already known: the prompt (inference_request.hpp:73-75), or, after a
        preemption, prompt plus the tokens generated so far.  A decoding request has exactly one
        pending token, the one it sampled last."""
        if self.state == RequestState.FINISHED:
            return False
        generated = len(self.generated_tokens)
        return generated == 0 or len(self.prompt_tokens) + generated - self.num_computed_tokens > 1

    def has_pending_input(self) -> bool:
        if self.unresolved and self.num_generated() >= self.max_new_tokens:
            return False       # the token still on the device is the last one allowed: it will not be fed
        return not self.is_finished() and self.num_computed_tokens < self.total_input_tokens()

    def can_generate_more(self) -> bool:
        return not self.is_finished() and self.num_generated() < self.max_new_tokens

    def all_tokens(self) -> list:
        return self.prompt_tokens + self.generated_tokens

    # ---- life cycle ----------------------------------------------------------------------------------------
    def start_running(self) -> None:
        self.state = RequestState.RUNNING
        if self.start_time is None:
            self.start_time = time.monotonic()

    def finish(self, reason: str = "stop") -> None:
        self.state = RequestState.FINISHED
        self.finish_reason = self.finish_reason or reason
        self.finish_time = time.monotonic()

    def preempt(self) -> None:
        """Its pages are gone: everything has to be computed again, from the first prompt token."""
        self.state = RequestState.WAITING
        self.num_computed_tokens = 0
        self.num_preemptions += 1

    # ---- chunk cutting (inference_request.hpp:145-184) -------------------------------------------------
    def pending_tokens(self) -> int:
        return 0 if self.is_finished() else self.total_input_tokens() - self.num_computed_tokens

    def get_next_chunk_size(self, chunk_size: int = 256) -> int:
        return min(chunk_size, self.pending_tokens())

    def get_next_chunk_tokens(self, chunk_size: int = 256) -> list:
        n = self.get_next_chunk_size(chunk_size)
        at, split = self.num_computed_tokens, len(self.prompt_tokens)
        if at >= split:                      # decoding: only generated tokens are touched
            return self.generated_tokens[at - split:at - split + n]
        if at + n <= split:
            return self.prompt_tokens[at:at + n]
        return self.prompt_tokens[at:] + self.generated_tokens[:at + n - split]

    def add_computed_tokens(self, count: int) -> None:
        if count <= 0:
            raise ValueError("Computed token count must be positive")
        if self.is_finished():
            raise RuntimeError("Request already finished")
        if self.num_computed_tokens + count > self.total_input_tokens():
            raise ValueError("Computed token count exceeds available inputs")
        self.num_computed_tokens += count

    def add_sampled_token(self, token: int, eos_token_ids) -> bool:
        """Append a sampled token; returns False when the request finished with it (130-143)."""
        if self.is_finished():
            return False
        self.generated_tokens.append(token)
        return self._after_token(token, eos_token_ids)

    def _after_token(self, token: int, eos_token_ids) -> bool:
        if token == -1:
            self.finish("invalid_token")
        elif not self.ignore_eos and token in eos_token_ids:
            self.finish("eos")
        elif self.num_generated() - self.unresolved >= self.max_new_tokens:
            self.finish("length")
        return not self.is_finished()

    # A token that was sampled on the device and is read back a step later: a place is kept for it at once, so
    # that the scheduler can plan the next step, and filled when the value arrives (oldest place first).
    PENDING_TOKEN = 0

    def add_pending_token(self) -> None:
        self.generated_tokens.append(self.PENDING_TOKEN)
        self.unresolved += 1

    def resolve_pending_token(self, token: int, eos_token_ids) -> bool:
        """Fill the oldest kept place; returns False when the request finished with this token."""
        self.generated_tokens[len(self.generated_tokens) - self.unresolved] = token
        self.unresolved -= 1
        return self._after_token(token, eos_token_ids)

    def drop_pending_tokens(self) -> None:
        """Places kept for tokens sampled after the one that ended the request."""
        while self.unresolved > 0:
            self.generated_tokens.pop()
            self.unresolved -= 1

    def resolved_tokens(self) -> list:
        return self.generated_tokens[:len(self.generated_tokens) - self.unresolved]
