"""Interfaces of the parts.

Part                 tensor_specs() -> [TensorSpec]; load(tensors: {name: Tensor})
TokenEmbedding(Part) forward(ids int32 [T]) -> [T, H];  table() -> the [V, H] tensor, or None
Head(Part)           forward(rows [R, H]) -> float32 logits [R, V];  ``tied``: load() is given
                     the embedding's table under the key None instead of a tensor of its own
Norm(Part)           forward(x) -> y;  add_forward(x, residual) -> (y, residual)
PositionEncoding     prepare(); rotary_table() -> Tensor | None; apply(q, k, positions)
Mixer(Part)          cache_spec() -> PagedKVSpec | StateSpec | None
                     forward(x [T, H], step, cache) -> [T, H]
FeedForward(Part)    forward(x [T, H]) -> [T, H]
Block                forward(hidden, residual, step, cache) -> (hidden, residual)

What a mixer or feed-forward returns, and what a block hands on as ``hidden``, is a
tensor or an ``ops.SplitSum`` (the float32 partial products of a matrix product
whose k was split, which the next norm adds while it loads them); the package's
kernels take either, and ``ops.as_tensor`` gives a plain tensor to code that needs
one.  The INPUT of a mixer or feed-forward is always a plain tensor (a norm's output).

``step`` is the step's ``StepBatch`` (tokens, positions, sequence boundaries,
state slots); ``cache`` is the view of the one cache the schedule entry names
(``CacheView``: the layer's page pool with its group's block table and slot
mapping, or the state array).  No part sees the model, the schedule, the
scheduler or another part's weights.
"""

from __future__ import annotations

from typing import Optional

import torch

from .spec import TensorSpec


class Part:
    kind = "?"

    def tensor_specs(self) -> list[TensorSpec]:
        return []

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        pass


class TokenEmbedding(Part):
    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    def table(self) -> Optional[torch.Tensor]:
        """The [vocabulary, hidden] tensor a tied head may share, or None."""
        return None


class Head(Part):
    tied = False      # True: ``load`` finds the embedding's table under the key None

    def forward(self, rows: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


class Norm(Part):
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    def add_forward(self, x: torch.Tensor, residual: torch.Tensor):
        raise NotImplementedError


class PositionEncoding(Part):
    def prepare(self) -> None:
        pass

    def rotary_table(self) -> Optional[torch.Tensor]:
        """float32 [max_positions, rotary_dim] = [cos | sin] for mixers that fuse
        the rotation into their own kernel, or None if this encoding is not a
        rotation."""
        return None


class Mixer(Part):
    def cache_spec(self):
        return None

    def forward(self, x: torch.Tensor, step, cache) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


class Block:
    kind = "?"

    def forward(self, hidden, residual, step, cache):
        raise NotImplementedError
