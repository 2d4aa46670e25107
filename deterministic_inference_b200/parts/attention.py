"""Grouped-query attention mixer over a paged cache.

qkv = x W_qkv^T (one product of the concatenated q, k, v weights, no bias); per
head RMSNorm of q and k with one weight [D] each (optional), the position
encoding's rotation, k and v written to the token's cache slot, attention of
every token over its sequence's cached keys (scale applied after the dot
product, causal by absolute position, optional window), output projection
(sid/model/qwen3.py:43-80, sid/model/loader.py:87-94).
"""

from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops
from .base import Mixer
from .registry import POSITION_ENCODINGS, register_mixer
from .spec import PagedKVSpec, PartSpec, TensorSpec


@register_mixer("gqa_attention")
class GQAAttention(Mixer):
    def __init__(self, ctx, prefix: str, hidden_size: int, num_heads: int, num_kv_heads: int,
                 head_dim: int, scale: float, position_encoding: PartSpec,
                 qk_norm_eps: Optional[float] = None, window: Optional[int] = None):
        if num_heads % num_kv_heads:
            raise ValueError(f"num_heads {num_heads} is not a multiple of num_kv_heads {num_kv_heads}")
        self.prefix = prefix
        self.hidden_size, self.num_heads = int(hidden_size), int(num_heads)
        self.num_kv_heads, self.head_dim = int(num_kv_heads), int(head_dim)
        self.scale = float(scale)
        self.qk_norm_eps = None if qk_norm_eps is None else float(qk_norm_eps)
        self.window = None if window is None else int(window)
        self.position_encoding = POSITION_ENCODINGS.build(position_encoding, ctx)
        self.w_qkv = self.w_o = self.q_norm = self.k_norm = None

    # -- weights
    def tensor_specs(self):
        p, h, d = self.prefix, self.hidden_size, self.head_dim
        specs = [
            TensorSpec(p + "q_proj.weight", (self.num_heads * d, h)),
            TensorSpec(p + "k_proj.weight", (self.num_kv_heads * d, h)),
            TensorSpec(p + "v_proj.weight", (self.num_kv_heads * d, h)),
            TensorSpec(p + "o_proj.weight", (h, self.num_heads * d)),
        ]
        if self.qk_norm_eps is not None:
            specs += [TensorSpec(p + "q_norm.weight", (d,), role="vector", init="one_plus_normal"),
                      TensorSpec(p + "k_norm.weight", (d,), role="vector", init="one_plus_normal")]
        return specs

    def load(self, tensors):
        p = self.prefix
        self.w_qkv = torch.cat([tensors[p + "q_proj.weight"], tensors[p + "k_proj.weight"],
                                tensors[p + "v_proj.weight"]], dim=0).contiguous()
        self.w_o = tensors[p + "o_proj.weight"]
        if self.qk_norm_eps is not None:
            self.q_norm = tensors[p + "q_norm.weight"]
            self.k_norm = tensors[p + "k_norm.weight"]
        self.position_encoding.prepare()

    # -- cache
    def cache_spec(self):
        return PagedKVSpec(self.num_kv_heads, self.head_dim, self.window)

    # -- step
    def forward(self, x, step, cache):
        # (one kernel for many bfloat16 rows of heads of 128, else the product and the q/k kernel)
        q = ops.qkv_project(
            x, self.w_qkv, self.num_heads, self.num_kv_heads, self.head_dim, self.q_norm, self.k_norm,
            self.qk_norm_eps if self.qk_norm_eps is not None else 0.0,
            self.position_encoding.rotary_table(), step.positions,
            cache.kv if cache.writes else None, cache.slot_mapping, cache.page_size)
        # (a decode-only step's attention may come back with its splits not yet merged; the
        # output projection then merges them while it loads its operand)
        o = ops.paged_attention(q, cache.kv, cache.attention_meta, self.scale, self.window, defer=True)
        return ops.linear(ops.merge_heads(o), self.w_o)
