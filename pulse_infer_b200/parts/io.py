"""The two ends of the model: the token embedding and the output head.

Reference parity: ``src/layer/embedding.cpp:132-153`` (row gather of int32 ids),
``src/model/qwen3/model.cpp:1322-1371`` (logits = x W^T with ``lm_head.weight``, or with the embedding
table when the model ties them).  The head here runs on the wanted rows only and returns 32-bit logits.
"""
from __future__ import annotations

import torch

from .. import ops
from .base import Part, TensorSpec, register_part


@register_part("embedding", "token_embedding")
class TokenEmbedding(Part):
    capturable = True       # see parts.base.Part.capturable
    def __init__(self, vocab_size: int, hidden_size: int):
        self.vocab_size = vocab_size
        self.hidden_size = hidden_size
        self.table: torch.Tensor | None = None

    def tensor_specs(self) -> dict:
        return {"weight": TensorSpec((self.vocab_size, self.hidden_size))}

    def load(self, tensors: dict, runtime) -> None:
        self.table = tensors["weight"].contiguous()
        self._tensors = {"table": self.table}

    def forward(self, tokens: torch.Tensor, ctx) -> torch.Tensor:
        return ops.embed(tokens, self.table)

    def tied_table(self) -> torch.Tensor:
        """[vocab, hidden]: what a head that shares the embedding's weights multiplies with."""
        return self.table


@register_part("head", "lm_head")
class LMHead(Part):
    capturable = True       # see parts.base.Part.capturable
    def __init__(self, vocab_size: int, hidden_size: int, tied: bool = False):
        self.vocab_size = vocab_size
        self.hidden_size = hidden_size
        self.tied = tied
        self.weight: torch.Tensor | None = None

    def tensor_specs(self) -> dict:
        # a tied model may still ship its own head; if it does, it is used (model.cpp:1009-1021)
        return {"weight": TensorSpec((self.vocab_size, self.hidden_size), optional=self.tied)}

    def load(self, tensors: dict, runtime) -> None:
        self.weight = tensors.get("weight")
        self._tensors = {} if self.weight is None else {"weight": self.weight}

    def first_weights(self):
        return self.weight

    def tie_to(self, table: torch.Tensor) -> None:
        self.weight = table

    def finish(self, embedding) -> None:
        """After loading: a tied head without a tensor of its own uses the embedding's table
        (``src/model/qwen3/model.cpp:1346-1371``); a head that ends up with nothing is an error (``model.cpp:1373``)."""
        if self.weight is None and self.tied:
            self.tie_to(embedding.tied_table())
        if self.weight is None:
            raise RuntimeError("lm_head is not initialized")

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        if self.weight is None:
            raise RuntimeError("lm_head is not initialized")  # model.cpp:1373
        # a step whose logits have a fixed home (recorded steps share one) writes them there
        home = getattr(ctx, "logits_out", None)
        out = home[:x.shape[0]] if home is not None and self.weight.dtype == torch.bfloat16 else None
        return ops.linear(x, self.weight, torch.float32, out=out)
