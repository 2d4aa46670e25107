"""bfloat16 matrix product y = x @ weight^T with float32 accumulation.

Few rows (decode steps, the head on the wanted rows): this package's tcgen05 kernel
(csrc/gemm_bf16.cu), which puts the weight rows on the tensor core's M axis and
streams the weight once, with a deterministic split of k when there are fewer
tiles than SMs.  Many rows (prompt portions): cuBLAS through ``torch.mm``, as the
reference hands every matrix product to the library (``F.linear``,
sid/model/qwen3.py:38).
"""

from __future__ import annotations

import os
from ctypes import c_int, c_longlong, c_void_p

import torch

# rows up to which the package's own kernel is used
MAX_ROWS = int(os.environ.get("DIB200_GEMM_MAX_ROWS", "128"))
_PARTIAL_FLOATS = 8 * 1024 * 1024      # split-k scratch per device (32 MiB)
_NUM_COUNTERS = 16384

_workspace: dict = {}


def _ws(device):
    ws = _workspace.get(device)
    if ws is None:
        ws = (torch.empty(_PARTIAL_FLOATS, dtype=torch.float32, device=device),
              torch.zeros(_NUM_COUNTERS, dtype=torch.int32, device=device),
              torch.cuda.get_device_properties(device).multi_processor_count)
        _workspace[device] = ws
    return ws


def status() -> int:
    """0, or 1 if a bounded wait inside the kernel ever ran out (synchronises)."""
    from .ops import _lib
    return int(_lib("gemm_bf16").dib_gemm_bf16_status())


def linear(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    from . import ops
    m, k = x.shape
    n = weight.shape[0]
    if m <= MAX_ROWS and k % 8 == 0 and k >= 8 and out_dtype in (torch.bfloat16, torch.float32) \
            and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0:
        partial, counters, sms = _ws(x.device)
        out = torch.empty(m, n, dtype=out_dtype, device=x.device)
        st = ops._lib("gemm_bf16").dib_gemm_bf16(
            ops._ptr(x), ops._ptr(weight), ops._ptr(out), c_int(m), c_int(n), c_int(k),
            c_int(1 if out_dtype == torch.float32 else 0), ops._ptr(partial),
            c_longlong(partial.numel()), ops._ptr(counters), c_int(counters.numel()), c_int(sms),
            ops._stream())
        ops._check(st, "linear(bfloat16)", f"M={m} N={n} K={k}")
        return out
    ops._launched(1)
    if out_dtype == torch.bfloat16:
        return torch.mm(x, weight.t())
    return torch.mm(x, weight.t(), out_dtype=out_dtype)
