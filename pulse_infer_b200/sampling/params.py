"""Per-request sampling options, with the names and meanings the reference's generation demo uses
(``demo/qwen3_infer.cpp:229-239,590-592``)."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0        # <= 0: greedy (qwen3_infer.cpp:277)
    top_k: int = 0                  # <= 0: all tokens (qwen3_infer.cpp:336)
    top_p: float = 0.0              # active only for 0 < p < 1 (qwen3_infer.cpp:395)
    presence_penalty: float = 0.0   # subtracted once from every token already in prompt or output (251-264)
    banned_tokens: tuple = ()       # never sampled (522-535)
    seed: int = 0                   # the draws of a request depend on (seed, index of the draw) only
    use_greedy: bool = False        # qwen3_infer.cpp:236

    @property
    def greedy(self) -> bool:
        return self.use_greedy or self.temperature <= 0.0

    @property
    def edits_logits(self) -> bool:
        return self.presence_penalty > 0.0 or bool(self.banned_tokens)
