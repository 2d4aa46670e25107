"""Rotary position encoding (rotate-half over the first ``rotary_dim`` dims of a
head): inv_freq_i = theta^(-i/(r/2)), angle = pos * inv_freq_i, all in float32;
the table [max_positions, rotary_dim] = [cos | sin] is built once
(sid/kernels/rope.py:41-48).  The rotation itself runs inside the attention
mixer's fused q/k kernel, which takes this table."""

from __future__ import annotations

import torch

from .base import PositionEncoding
from .registry import register_position_encoding


@register_position_encoding("rope")
class RotaryEmbedding(PositionEncoding):
    def __init__(self, ctx, head_dim: int, rotary_dim: int, theta: float, max_positions: int):
        if rotary_dim % 2 or rotary_dim > head_dim:
            raise ValueError(f"rotary_dim {rotary_dim} must be even and at most head_dim {head_dim}")
        self.head_dim, self.rotary_dim = int(head_dim), int(rotary_dim)
        self.theta, self.max_positions = float(theta), int(max_positions)
        self.ctx = ctx
        self._table = None

    def prepare(self):
        key = ("rope", self.rotary_dim, self.theta, self.max_positions)
        table = self.ctx.shared.get(key)
        if table is None:
            half = self.rotary_dim // 2
            dev = self.ctx.device
            inv_freq = 1.0 / (self.theta ** (torch.arange(0, half, dtype=torch.float32, device=dev) / half))
            pos = torch.arange(self.max_positions, dtype=torch.float32, device=dev)
            freqs = torch.outer(pos, inv_freq)
            table = torch.cat([freqs.cos(), freqs.sin()], dim=-1).contiguous()
            self.ctx.shared[key] = table
        self._table = table

    def rotary_table(self):
        if self._table is None:
            self.prepare()
        return self._table


@register_position_encoding("none")
class NoPositionEncoding(PositionEncoding):
    """No position encoding: q and k go to attention as projected."""

    def __init__(self, ctx, **_):
        pass
