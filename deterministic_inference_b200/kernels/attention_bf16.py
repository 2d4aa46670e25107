"""bfloat16 tensor-core attention over the paged cache (prefill/extend and
split-KV decode).  ``supports`` says whether the kernels take a shape; shapes
they refuse run on the generic kernel."""

from __future__ import annotations


def supports(num_heads: int, num_kv_heads: int, head_dim: int, page_size: int) -> bool:
    return False


def run(q, out, kv_cache, meta, scale: float, window: int) -> None:
    raise NotImplementedError
