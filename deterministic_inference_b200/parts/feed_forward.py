"""Dense gated feed-forward: down( act(gate(x)) * up(x) ), no biases; gate and up
are one product of the concatenated weights, gate first
(sid/model/qwen3.py:82-86, sid/model/loader.py:97-101)."""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import FeedForward
from .registry import register_feed_forward
from .spec import TensorSpec


@register_feed_forward("gated_mlp")
class GatedMLP(FeedForward):
    def __init__(self, ctx, prefix: str, hidden_size: int, intermediate_size: int,
                 activation: str = "silu"):
        if activation != "silu":
            raise ValueError(f"gated_mlp: activation {activation!r} has no kernel (only 'silu')")
        self.prefix = prefix
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        self.w_gate_up = self.w_down = None

    def tensor_specs(self):
        p, h, i = self.prefix, self.hidden_size, self.intermediate_size
        return [TensorSpec(p + "gate_proj.weight", (i, h)), TensorSpec(p + "up_proj.weight", (i, h)),
                TensorSpec(p + "down_proj.weight", (h, i))]

    def load(self, tensors):
        p = self.prefix
        self.w_gate_up = torch.cat([tensors[p + "gate_proj.weight"], tensors[p + "up_proj.weight"]],
                                   dim=0).contiguous()
        self.w_down = tensors[p + "down_proj.weight"]

    def forward(self, x):
        return ops.linear(ops.gated_linear(x, self.w_gate_up), self.w_down)
