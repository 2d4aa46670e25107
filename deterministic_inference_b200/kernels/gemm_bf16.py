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
from ctypes import byref, c_float, c_int, c_longlong, c_void_p

import torch

# Rows up to which the few-rows kernel (swap-AB, split of k) is used; products of more rows go
# to the many-rows kernel or the library.  ``set_library_products(False)`` sends every product
# to the few-rows kernel, whose order of summation does not depend on the number of rows: a
# token's bits are then the same whatever else the step holds (the library's algorithm depends
# on the shape).  64: the split of k is the decode step's (a function of the layer's sizes
# alone), and its float32 partial sums grow with the rows: from 65 rows on they cost more than
# the other kernels' few tiles do (0.6B sizes on B200: a prompt of 128 tokens 1.60 against
# 1.95 ms, decode at batch 96 / 128 17,800 / 20,200 against 16,500 / 19,100 tokens a second;
# batch 48 unchanged; a line at 48 is 3 % slower at batch 56 and 64, one at 32 slower at 48).
OWN_KERNEL_ROWS = int(os.environ.get("DIB200_GEMM_MAX_ROWS", "64"))
MAX_ROWS = OWN_KERNEL_ROWS
# DIB200_GATED=0/1 (read once): never / always the gate in the product's epilogue
GATED = os.environ.get("DIB200_GATED")


# Products of more than MAX_ROWS rows (``EngineConfig.large_products``; DIB200_LARGE_PRODUCTS
# in the environment, read once, gives the default):
#   "library"  cuBLAS through torch.mm, as all of the reference's products;
#   "own"      the package's persistent tcgen05 kernel for many rows (csrc/gemm_bf16_large.cu),
#              which adds up all of k in one pass, so a row's bits do not depend on how many
#              rows (above MAX_ROWS) there are, and which the first step of a new length does
#              not pay a library's kernel loading for;
#   "auto"     that kernel where it carries the gate of a gated feed-forward in its epilogue
#              (one kernel and no [gate | up] tensor instead of two), the library elsewhere:
#              the fastest replayed prompt step on B200 (0.6B sizes, 2,048 tokens, per layer:
#              61.7 us against 65.5 all-library and 78.2 all-own).
LARGE_PRODUCTS = os.environ.get("DIB200_LARGE_PRODUCTS", "auto")


def set_large_products(how: str) -> None:
    global LARGE_PRODUCTS
    if how not in ("library", "own", "auto"):
        raise ValueError(f"large_products must be 'library', 'own' or 'auto', got {how!r}")
    LARGE_PRODUCTS = how


def set_library_products(on: bool) -> None:
    global MAX_ROWS
    MAX_ROWS = OWN_KERNEL_ROWS if on else 1 << 30


def linear_large(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype):
    """x [M, K] @ weight[N, K]^T by the package's kernel for many rows, or None if the
    shape is not one it takes."""
    from . import ops
    m, k = x.shape
    n = weight.shape[0]
    if not (k % 8 == 0 and k >= 8 and n % (4 if out_dtype == torch.float32 else 8) == 0
            and out_dtype in (torch.bfloat16, torch.float32)
            and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0):
        return None
    out = torch.empty(m, n, dtype=out_dtype, device=x.device)
    st = ops._lib("gemm_bf16_large").dib_gemm_bf16_large(
        ops._ptr(x), ops._ptr(weight), ops._ptr(out), c_int(m), c_int(n), c_int(k),
        c_int(1 if out_dtype == torch.float32 else 0), c_int(_sms(x.device)), ops._stream())
    ops._check(st, "linear(bfloat16, many rows)", f"M={m} N={n} K={k}")
    return out


def gated_linear_large(x: torch.Tensor, w_gate_up: torch.Tensor):
    """silu(x @ w_gate^T) * (x @ w_up^T) in the many-rows kernel's epilogue, or None."""
    from . import ops
    m, k = x.shape
    i = w_gate_up.shape[0] // 2
    if not (k % 8 == 0 and k >= 8 and i % 8 == 0 and w_gate_up.shape[0] == 2 * i
            and x.data_ptr() % 16 == 0 and w_gate_up.data_ptr() % 16 == 0):
        return None
    out = torch.empty(m, i, dtype=torch.bfloat16, device=x.device)
    st = ops._lib("gemm_bf16_large").dib_gemm_bf16_large_gated(
        ops._ptr(x), ops._ptr(w_gate_up), ops._ptr(out), c_int(m), c_int(i), c_int(k),
        c_int(_sms(x.device)), ops._stream())
    ops._check(st, "gated_linear(bfloat16, many rows)", f"M={m} I={i} K={k}")
    return out



# DIB200_QKV_EPILOGUE=0 (read once): q/k norm, rotation and cache write stay a kernel of their own
QKV_EPILOGUE = os.environ.get("DIB200_QKV_EPILOGUE", "1") != "0"


def qkv_large(x: torch.Tensor, w_qkv: torch.Tensor, num_heads: int, num_kv_heads: int, q_norm_weight,
              k_norm_weight, eps: float, cos_sin, positions, kv_cache, slot_mapping, page_size: int):
    """q [M, Hq, 128] of the fused projection with q/k norm, rotation and cache write in the
    many-rows product's epilogue, or None where that kernel does not run the step's
    projection (few rows, the library for all large products, a shape it refuses)."""
    from . import ops
    m, k = x.shape
    if not QKV_EPILOGUE or m <= MAX_ROWS or LARGE_PRODUCTS not in ("own", "auto"):
        return None
    n = (num_heads + 2 * num_kv_heads) * 128
    if w_qkv.shape[0] != n or w_qkv.shape[1] != k or k % 8 != 0 or k < 8 or w_qkv.dtype != torch.bfloat16 \
            or kv_cache.dtype != torch.bfloat16 or x.data_ptr() % 16 or w_qkv.data_ptr() % 16 \
            or kv_cache.data_ptr() % 16 or tuple(kv_cache.shape[1:]) != (2, num_kv_heads, page_size, 128):
        return None
    for w in (q_norm_weight, k_norm_weight):
        if w is not None and (w.dtype != torch.float32 or w.shape[0] != 128):
            return None
    if positions.dtype != torch.int32 or slot_mapping.dtype != torch.int32 or positions.shape[0] < m \
            or slot_mapping.shape[0] < m:
        return None
    q = torch.empty(m, num_heads, 128, dtype=torch.bfloat16, device=x.device)
    st = ops._lib("gemm_bf16_large").dib_gemm_bf16_large_qkv(
        ops._ptr(x), ops._ptr(w_qkv), ops._ptr(q), c_int(m), c_int(k), c_int(num_heads), c_int(num_kv_heads),
        ops._ptr(q_norm_weight), ops._ptr(k_norm_weight), c_float(eps), ops._ptr(cos_sin),
        c_int(cos_sin.shape[0] if cos_sin is not None else 0), ops._ptr(positions), ops._ptr(slot_mapping),
        ops._ptr(kv_cache), c_longlong(kv_cache.shape[0]), c_int(page_size), c_int(_sms(x.device)), ops._stream())
    ops._check(st, "qkv projection(bfloat16, many rows)", f"M={m} K={k} heads {num_heads}/{num_kv_heads}")
    return q


def force_large_shape(shape: int) -> None:
    """Measurement and test switch of the many-rows kernel: tiles of 128 x 128 (0) or 128 x 256
    (1) by one CTA, or of 256 x 256 by a pair of CTAs (2), whatever the sizes; -1: the kernel
    library's own choice.  The result's bits are the same with all three."""
    from . import ops
    ops._lib("gemm_bf16_large").dib_gemm_bf16_large_force_shape(c_int(shape))


_sm_count: dict = {}


def _sms(device) -> int:
    n = _sm_count.get(device)
    if n is None:
        n = torch.cuda.get_device_properties(device).multi_processor_count
        _sm_count[device] = n
    return n


def configure(cluster: int = -1, forced_splits: int = -1) -> None:
    """Measurement and test switches of the kernel library (negative: leave as it is):
    ``cluster`` 0/1: the CTAs of a tile add their partial tiles up as a thread-block
    cluster; ``forced_splits`` n >= 1: split k n ways, 0: the cost model's choice."""
    from .ops import _lib
    _lib("gemm_bf16").dib_gemm_bf16_configure(c_int(cluster), c_int(forced_splits))


def status() -> int:
    """0, or 1 if a bounded wait inside the kernel ever ran out (synchronises)."""
    from .ops import _lib
    return int(_lib("gemm_bf16").dib_gemm_bf16_status())


def plan(m: int, n: int, k: int, device) -> tuple:
    """(tokens per tile, k-blocks per split, splits) the kernel uses for these sizes."""
    from .ops import _lib
    bn, per, splits = c_int(), c_int(), c_int()
    _lib("gemm_bf16").dib_gemm_bf16_plan(c_int(m), c_int(n), c_int(k), c_int(_sms(device)),
                                         byref(bn), byref(per), byref(splits))
    return bn.value, per.value, splits.value


def linear(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype, allow_split: bool = True):
    """x [M, K] @ weight[N, K]^T.  Returns a tensor, or, when the kernel splits k and
    ``allow_split``, an ``ops.SplitSum`` of its float32 partial products."""
    from . import ops
    m, k = x.shape
    n = weight.shape[0]
    if m <= MAX_ROWS and k % 8 == 0 and k >= 8 and out_dtype in (torch.bfloat16, torch.float32) \
            and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0:
        lib = ops._lib("gemm_bf16")
        splits = plan(m, n, k, x.device)[2] if allow_split else 1
        fp32 = c_int(1 if out_dtype == torch.float32 else 0)
        # a split of k that the tile's cluster adds up itself comes out finished
        if splits > 1 and lib.dib_gemm_bf16_cluster_reduces(c_int(n), c_int(k), c_int(_sms(x.device))):
            splits = 1
        if splits > 1:
            parts = torch.empty(splits, m, n, dtype=torch.float32, device=x.device)
            st = lib.dib_gemm_bf16(ops._ptr(x), ops._ptr(weight), c_void_p(0), c_int(m), c_int(n),
                                   c_int(k), fp32, ops._ptr(parts), c_int(_sms(x.device)),
                                   ops._stream())
            ops._check(st, "linear(bfloat16)", f"M={m} N={n} K={k}")
            return ops.SplitSum(parts, out_dtype)
        out = torch.empty(m, n, dtype=out_dtype, device=x.device)
        st = lib.dib_gemm_bf16(ops._ptr(x), ops._ptr(weight), ops._ptr(out), c_int(m), c_int(n),
                               c_int(k), fp32, c_void_p(0), c_int(_sms(x.device)), ops._stream())
        ops._check(st, "linear(bfloat16)", f"M={m} N={n} K={k}")
        return out
    if LARGE_PRODUCTS == "own":
        out = linear_large(x, weight, out_dtype)
        if out is not None:
            return out
    ops._launched(1)
    if out_dtype == torch.bfloat16:
        return torch.mm(x, weight.t())
    return torch.mm(x, weight.t(), out_dtype=out_dtype)


def linear_of_deferred(x, weight: torch.Tensor, out_dtype: torch.dtype):
    """x @ weight^T for an ``ops.GatedSplit`` or ``ops.SplitAttention`` x: the kernel makes
    its token operand from the partial results while its weights arrive.  None if the shape
    is not one the kernel takes (the caller then materialises x)."""
    from . import ops
    m, k = x.shape
    n = weight.shape[0]
    if not (m <= min(MAX_ROWS, 128) and k % 8 == 0 and out_dtype in (torch.bfloat16, torch.float32)
            and weight.data_ptr() % 16 == 0 and weight.is_contiguous()):
        return None
    lib = ops._lib("gemm_bf16")
    splits = plan(m, n, k, weight.device)[2]
    fp32 = c_int(1 if out_dtype == torch.float32 else 0)
    if isinstance(x, ops.GatedSplit):
        g = x.gate_up.parts
        pro, args = 1, (ops._ptr(g), c_int(g.shape[0]), c_longlong(g.shape[1] * g.shape[2]),
                        c_void_p(0), c_void_p(0), c_void_p(0), c_int(0), c_int(0), c_int(0))
    else:
        if x.head_dim % 4:
            return None
        pro, args = 2, (c_void_p(0), c_int(0), c_longlong(0), ops._ptr(x.part_o), ops._ptr(x.part_lse),
                        ops._ptr(x.seq_lens), c_int(x.max_splits), c_int(x.head_dim), c_int(x.window))
    parts = out = None
    if splits > 1:
        parts = torch.empty(splits, m, n, dtype=torch.float32, device=weight.device)
    else:
        out = torch.empty(m, n, dtype=out_dtype, device=weight.device)
    st = lib.dib_gemm_bf16_operand(c_int(pro), ops._ptr(weight), ops._ptr(out), c_int(m), c_int(n), c_int(k),
                                   fp32, ops._ptr(parts), c_int(_sms(weight.device)), *args, ops._stream())
    if st == -2:
        return None
    ops._check(st, "linear(bfloat16, operand made in the kernel)", f"M={m} N={n} K={k}")
    return ops.SplitSum(parts, out_dtype) if parts is not None else out


def gated_linear(x: torch.Tensor, w_gate_up: torch.Tensor):
    """silu(x @ w_gate^T) * (x @ w_up^T) for w_gate_up = [w_gate ; w_up] ([2I, K]) in one
    kernel (the gate happens in the product's epilogue), or None if the shape does not
    allow it (the caller then runs the product and the gate separately)."""
    from . import ops
    m, k = x.shape
    i = w_gate_up.shape[0] // 2
    if m > MAX_ROWS:
        return gated_linear_large(x, w_gate_up) if LARGE_PRODUCTS in ("own", "auto") else None
    # one CTA per 64 features and no split of k: worth it when those CTAs fill whole waves
    # of the GPU about as well as the split product does (the kernel's own estimate; 0.6B
    # shape, 48 tiles: 1.458 ms per step against 1.435 ms with the split product and the
    # separate gate).  ``GATED`` forces the choice.
    forced = GATED
    if forced == "0" or (forced != "1" and not ops._lib("gemm_bf16").dib_gemm_bf16_gated_pays(
            c_int(i), c_int(k), c_int(_sms(x.device)))):
        return None
    if not (m <= MAX_ROWS and k % 8 == 0 and k >= 8 and i % 64 == 0 and w_gate_up.shape[0] == 2 * i
            and x.data_ptr() % 16 == 0 and w_gate_up.data_ptr() % 16 == 0):
        return None
    out = torch.empty(m, i, dtype=torch.bfloat16, device=x.device)
    st = ops._lib("gemm_bf16").dib_gemm_bf16_gated(ops._ptr(x), ops._ptr(w_gate_up), ops._ptr(out),
                                                   c_int(m), c_int(i), c_int(k), c_int(_sms(x.device)), ops._stream())
    ops._check(st, "gated_linear(bfloat16)", f"M={m} I={i} K={k}")
    return out
