"""Registries from a part's kind to its class.

``register_mixer("gqa_attention")(cls)`` makes the kind available to every
plan.  A part class is built with ``cls(ctx=BuildContext, **spec.params)`` and
knows nothing of the model it sits in.  Registering a new kind needs no change
to any file of this package.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch

from .spec import PartSpec


@dataclass
class BuildContext:
    """What a part may know of its surroundings: the engine dtype and device, and
    a place where parts built from equal parameters can share what they prepare
    (the rotary table of all layers is one tensor)."""

    dtype: torch.dtype
    device: torch.device
    shared: dict = field(default_factory=dict)


class Registry:
    def __init__(self, what: str):
        self.what = what
        self._kinds: dict[str, type] = {}

    def register(self, kind: str):
        def deco(cls):
            self._kinds[kind] = cls
            cls.kind = kind
            return cls
        return deco

    def build(self, spec: PartSpec, ctx: BuildContext):
        if spec.kind not in self._kinds:
            raise KeyError(f"unknown {self.what} kind {spec.kind!r}; registered: {sorted(self._kinds)}")
        return self._kinds[spec.kind](ctx=ctx, **spec.params)

    def create(self, spec: PartSpec, ctx: BuildContext, **built):
        """Like ``build`` with already built parts passed beside the parameters
        (a block receives its mixer, feed-forward and norms)."""
        if spec.kind not in self._kinds:
            raise KeyError(f"unknown {self.what} kind {spec.kind!r}; registered: {sorted(self._kinds)}")
        return self._kinds[spec.kind](ctx=ctx, **built, **spec.params)

    def kinds(self) -> list[str]:
        return sorted(self._kinds)


EMBEDDINGS = Registry("embedding")
HEADS = Registry("head")
MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
NORMS = Registry("norm")
POSITION_ENCODINGS = Registry("position encoding")
BLOCKS = Registry("block")

register_embedding = EMBEDDINGS.register
register_head = HEADS.register
register_mixer = MIXERS.register
register_feed_forward = FEED_FORWARDS.register
register_norm = NORMS.register
register_position_encoding = POSITION_ENCODINGS.register
register_block = BLOCKS.register
