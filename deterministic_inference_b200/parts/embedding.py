"""The two ends of the decoder as parts: the token embedding (a row gather,
sid/model/qwen3.py:93) and the head on the wanted rows (a matrix product whose float32
accumulator is the logits, sid/model/qwen3.py:113-115).  The head has a weight of its own
or shares the embedding's table (sid/model/loader.py:74-82)."""

from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops
from .base import Head, TokenEmbedding
from .registry import register_embedding, register_head
from .spec import TensorSpec


@register_embedding("token_embedding")
class GatherEmbedding(TokenEmbedding):
    def __init__(self, ctx, name: str, vocab_size: int, hidden_size: int):
        self.name, self.vocab_size, self.hidden_size = name, int(vocab_size), int(hidden_size)
        self.weight = None

    def tensor_specs(self):
        return [TensorSpec(self.name, (self.vocab_size, self.hidden_size), role="table")]

    def load(self, tensors):
        self.weight = tensors[self.name]

    def table(self):
        return self.weight

    def forward(self, ids):
        return ops.embedding(ids, self.weight)


@register_head("linear_head")
class LinearHead(Head):
    """logits = rows @ W^T in float32.  ``name`` None: W is the embedding's table."""

    def __init__(self, ctx, name: Optional[str], vocab_size: int, hidden_size: int):
        self.name, self.vocab_size, self.hidden_size = name, int(vocab_size), int(hidden_size)
        self.tied = name is None
        self.weight = None

    def tensor_specs(self):
        return [] if self.tied else [TensorSpec(self.name, (self.vocab_size, self.hidden_size))]

    def load(self, tensors):
        self.weight = tensors[None] if self.tied else tensors[self.name]
        if self.weight is None or tuple(self.weight.shape) != (self.vocab_size, self.hidden_size):
            raise ValueError(f"head: no [{self.vocab_size}, {self.hidden_size}] table to share or load")

    def forward(self, rows):
        # logits leave as a plain tensor (the product may come as split-k partials)
        return ops.as_tensor(ops.linear(rows, self.weight, out_dtype=torch.float32))
