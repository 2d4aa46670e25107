"""RMSNorm part: y = x / sqrt(mean(x^2) + eps) * w, float32 arithmetic, eps
inside the root, the weight multiplies directly (sid/kernels/rmsnorm.py:14-24).
``add_forward`` is the fused residual form: residual += x, then the norm of the
unrounded sum, both in place (sid/kernels/rmsnorm.py:27-42)."""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import Norm
from .registry import register_norm
from .spec import TensorSpec


@register_norm("rms_norm")
class RMSNorm(Norm):
    def __init__(self, ctx, name: str, size: int, eps: float):
        self.name, self.size, self.eps = name, int(size), float(eps)
        self.weight = None

    def tensor_specs(self):
        return [TensorSpec(self.name, (self.size,), role="vector", init="one_plus_normal")]

    def load(self, tensors):
        self.weight = tensors[self.name]

    def forward(self, x):
        return ops.rms_norm(x, self.weight, self.eps)

    def add_forward(self, x, residual):
        return ops.add_rms_norm(x, residual, self.weight, self.eps)
