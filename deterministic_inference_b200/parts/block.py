"""Arrangement of a layer's parts and of the residual stream.

``pre_norm``: norm -> mixer -> norm -> feed-forward, the residual carried beside
the hidden state: the first norm site takes the embedding as the residual, every
later one adds the previous part's output to the residual and norms the sum
(sid/model/qwen3.py:94-108)."""

from __future__ import annotations

from .base import Block
from .registry import register_block


@register_block("pre_norm")
class PreNormBlock(Block):
    def __init__(self, ctx, mixer, feed_forward, mixer_norm, feed_forward_norm):
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm, self.feed_forward_norm = mixer_norm, feed_forward_norm

    def forward(self, hidden, residual, step, cache):
        if residual is None:
            residual = hidden
            hidden = self.mixer_norm.forward(hidden)
        else:
            hidden, residual = self.mixer_norm.add_forward(hidden, residual)
        hidden = self.mixer.forward(hidden, step, cache)
        hidden, residual = self.feed_forward_norm.add_forward(hidden, residual)
        hidden = self.feed_forward.forward(hidden)
        return hidden, residual
