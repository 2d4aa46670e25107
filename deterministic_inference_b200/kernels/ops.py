"""Python side of the CUDA kernels: argument checks and launches.

Every function takes CUDA tensors, checks dtype, shape and contiguity on the
host, and launches the hand-written kernel on the current stream.  There is no
CPU path and no library fallback: a tensor that is not on a CUDA device raises
``KernelError``, and a missing or unbuildable library raises
``KernelBuildError``.  The one library call is the bfloat16 matrix product of
``linear`` (cuBLAS through ``torch.mm``) for shapes the package's own tcgen05
kernel does not take; the reference uses the library for every matrix product
(sid/model/qwen3.py:38).

The parts call these functions through the module (``ops.rms_norm(...)``), so a
test can substitute plain PyTorch restatements to exercise the engine's host
logic on a machine without a GPU; the package itself never does.
"""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from . import build


class KernelError(RuntimeError):
    pass


_STATUS = {
    -1: "unsupported dtype",
    -2: "a size this kernel refuses",
    -3: "misaligned pointer",
    -4: "kernel launch failed",
    -5: "a bounded wait inside the kernel ran out",
}

_DT = {torch.float32: 0, torch.bfloat16: 1}


def _ptr(t):
    return c_void_p(t.data_ptr()) if t is not None else c_void_p(0)


try:
    _raw_stream = torch._C._cuda_getCurrentRawStream      # a plain integer handle, cheap
except AttributeError:                                     # pragma: no cover
    _raw_stream = None


def _stream():
    """Handle of the current CUDA stream of the current device."""
    if _raw_stream is not None:
        return c_void_p(_raw_stream(torch.cuda.current_device()))
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _check(status: int, what: str, detail: str = "", kernels: int = 1):
    global launch_count
    launch_count += kernels
    if status != 0:
        raise KernelError(f"{what}: {_STATUS.get(status, status)}{(' — ' + detail) if detail else ''}")


def _need(t: torch.Tensor, name: str, dtype=None, ndim=None):
    if not isinstance(t, torch.Tensor):
        raise KernelError(f"{name} must be a tensor")
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor: this package has no CPU path")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous (shape {tuple(t.shape)}, stride {t.stride()})")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    if ndim is not None and t.dim() != ndim:
        raise KernelError(f"{name} must have {ndim} dims, got shape {tuple(t.shape)}")


def _dt(t: torch.Tensor, name: str) -> int:
    if t.dtype not in _DT:
        raise KernelError(f"{name}: dtype {t.dtype} is not supported (float32 or bfloat16)")
    return _DT[t.dtype]


_libs: dict[str, ctypes.CDLL] = {}

# Kernels launched by this module since import (this package's own kernels plus
# the library matrix products it calls); benchmarks read differences of it.
launch_count = 0


def _launched(n: int = 1) -> None:
    global launch_count
    launch_count += n


def _lib(name: str) -> ctypes.CDLL:
    lib = _libs.get(name)
    if lib is None:
        lib = build.load_library(name)
        _libs[name] = lib
    return lib


# Libraries whose kernels have bounded waits: name -> (read, clear) of its error word.
_STATUS_FUNCTIONS = {
    "gemm_bf16": ("dib_gemm_bf16_status", "dib_gemm_bf16_status_clear"),
    "gemm_bf16_large": ("dib_gemm_bf16_large_status", "dib_gemm_bf16_large_status_clear"),
    "attention_bf16": ("dib_attention_bf16_status", "dib_attention_bf16_status_clear"),
    "attention_prefill_tc": ("dib_attention_prefill_tc_status", "dib_attention_prefill_tc_status_clear"),
}
_extra_status: dict = {}


def register_kernel_status(name: str, read, clear) -> None:
    """Add the error word of a library loaded from outside this module: ``read()`` gives 0
    or the code of a wait that ran out, ``clear()`` sets it back to 0."""
    _extra_status[name] = (read, clear)


def kernel_status() -> dict:
    """The error words of the libraries with bounded waits that have been loaded: name ->
    0, or the code of a wait that ran out (the results of that launch are not valid).
    Reading them synchronises with the device."""
    out = {}
    for name, (read, _) in _STATUS_FUNCTIONS.items():
        lib = _libs.get(name)
        if lib is not None:
            out[name] = int(getattr(lib, read)())
    for name, (read, _) in _extra_status.items():
        out[name] = int(read())
    return out


def clear_kernel_status() -> None:
    """Set every error word back to 0."""
    for name, (_, clear) in _STATUS_FUNCTIONS.items():
        lib = _libs.get(name)
        if lib is not None:
            getattr(lib, clear)()
    for _, clear in _extra_status.values():
        clear()


def check_kernel_status() -> None:
    """Raise ``KernelError`` if a bounded wait inside a kernel ran out since the last check.
    The words are cleared first, so the failure is reported once and later work is judged
    on its own."""
    bad = {k: v for k, v in kernel_status().items() if v != 0}
    if bad:
        clear_kernel_status()
        raise KernelError(f"a bounded wait inside a kernel ran out (library: code): {bad}; results of "
                          "the steps since the last check are not valid")


# ---------------------------------------------------------------- deferred sums

class SplitSum:
    """A matrix that exists as ``S`` float32 partial products of a split-k matrix
    product, ``parts[s]`` of shape [rows, cols], not yet added.  The kernels that
    read a projection output (residual-add + norm, q/k norm, SiLU gate) take it as
    it is and add the partials in split order while they load, rounding the sum to
    ``dtype`` as a stored product would be; anything else gets a plain tensor from
    ``as_tensor``.  ``hidden`` handed from a block to the next may be one."""

    def __init__(self, parts: torch.Tensor, dtype: torch.dtype):
        self.parts, self.dtype = parts, dtype

    @property
    def shape(self):
        return self.parts.shape[1:]

    @property
    def device(self):
        return self.parts.device

    @property
    def splits(self) -> int:
        return self.parts.shape[0]

    def tensor(self) -> torch.Tensor:
        s, m, n = self.parts.shape
        out = torch.empty(m, n, dtype=self.dtype, device=self.parts.device)
        if (m * n) % 4 == 0:
            st = _lib("elementwise").dib_sum_split(_ptr(self.parts), c_int(s), c_longlong(m * n),
                                                   _ptr(out), c_longlong(m * n),
                                                   c_int(_DT[self.dtype]), _stream())
            _check(st, "sum_split")
            return out
        _launched(1)
        acc = self.parts[0].clone()
        for i in range(1, s):          # split order
            acc += self.parts[i]
        return acc.to(self.dtype)


# Rows up to which the gate of a gated feed-forward is left to the product that follows
# (``GatedSplit``).  The product then stages the partial products of its columns in shared
# memory; with more than a few rows that costs more than the separate gate kernel (B200,
# width 1,024 / 3,072: 6.2 against 7.2 us for both products at 1 row, 8.2 against 7.5 us at 8);
# and with a wide feed-forward too (width 4,096 / 12,288: a decode step of one request 5 %
# slower with it), so it is limited to feed-forwards up to GATE_IN_PRODUCT_WIDTH wide.
GATE_IN_PRODUCT_ROWS = 2
GATE_IN_PRODUCT_WIDTH = 4096


class GatedSplit:
    """silu(gate) * up that is not computed yet: the [gate | up] product exists as the
    split-k partial products ``gate_up`` (a ``SplitSum``, [rows, 2I]).  The matrix product
    that follows makes its operand from them while it loads (``linear``); anything else gets
    the tensor [rows, I] from ``tensor()`` (the gate kernel that reads partials)."""

    def __init__(self, gate_up: SplitSum):
        self.gate_up = gate_up
        self.dtype = gate_up.dtype

    @property
    def shape(self):
        rows, two_i = self.gate_up.shape
        return torch.Size((rows, two_i // 2))

    @property
    def device(self):
        return self.gate_up.device

    def tensor(self) -> torch.Tensor:
        return silu_mul(self.gate_up)


class SplitAttention:
    """The output of the split-KV decode attention before its splits are merged:
    ``part_o`` float32 [sequences, heads, splits, head_dim], ``part_lse`` [sequences, heads,
    splits], the sequences' lengths on the device and the window.  Its logical shape is
    [sequences, heads * head_dim].  The output projection merges while it loads its
    operand (``linear``); ``tensor()`` runs the merge kernel."""

    def __init__(self, part_o, part_lse, seq_lens, num_seqs: int, window: int, dtype):
        self.part_o, self.part_lse, self.seq_lens = part_o, part_lse, seq_lens
        self.num_seqs, self.window, self.dtype = num_seqs, window, dtype
        _, self.num_heads, self.max_splits, self.head_dim = part_o.shape

    @property
    def shape(self):
        return torch.Size((self.num_seqs, self.num_heads * self.head_dim))

    @property
    def device(self):
        return self.part_o.device

    def tensor(self) -> torch.Tensor:
        out = torch.empty(self.num_seqs, self.num_heads, self.head_dim, dtype=self.dtype,
                          device=self.part_o.device)
        st = _lib("attention_bf16").dib_decode_attention_merge(
            _ptr(self.part_o), _ptr(self.part_lse), _ptr(self.seq_lens), _ptr(out), c_int(self.num_seqs),
            c_int(self.max_splits), c_int(self.num_heads), c_int(self.head_dim), c_int(self.window),
            _stream())
        _check(st, "decode_attention_merge")
        return out.view(self.num_seqs, self.num_heads * self.head_dim)


_DEFERRED = (SplitSum, GatedSplit, SplitAttention)


def as_tensor(x):
    """A plain tensor, whatever ``x`` is."""
    return x.tensor() if isinstance(x, _DEFERRED) else x


def merge_heads(o):
    """Attention output [T, heads, head_dim] as the output projection's operand
    [T, heads * head_dim] (a ``SplitAttention`` has that shape already)."""
    if isinstance(o, SplitAttention):
        return o
    return o.view(o.shape[0], o.shape[1] * o.shape[2])


# ---------------------------------------------------------------- embedding

def embedding(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """out[t] = table[ids[t]]; ids int32 [T], table [V, H]."""
    _need(ids, "ids", torch.int32, 1)
    _need(table, "table", None, 2)
    out = torch.empty(ids.shape[0], table.shape[1], dtype=table.dtype, device=table.device)
    st = _lib("elementwise").dib_embedding(
        _ptr(table), _ptr(ids), _ptr(out), c_int(ids.shape[0]), c_int(table.shape[1]),
        c_int(table.shape[0]), c_int(_dt(table, "table")), _stream())
    _check(st, "embedding")
    return out


def patch_token_ids(input_ids: torch.Tensor, patch_dst: torch.Tensor, patch_src: torch.Tensor,
                    prev_tokens: torch.Tensor) -> None:
    """input_ids[patch_dst[i]] = prev_tokens[patch_src[i]] where patch_dst[i] >= 0 (all
    int32): the tokens the previous step sampled become inputs on the device."""
    for t, n in ((input_ids, "input_ids"), (patch_dst, "patch_dst"), (patch_src, "patch_src"),
                 (prev_tokens, "prev_tokens")):
        _need(t, n, torch.int32, 1)
    st = _lib("elementwise").dib_patch_ids(_ptr(input_ids), _ptr(patch_dst), _ptr(patch_src),
                                           _ptr(prev_tokens), c_int(patch_dst.shape[0]),
                                           c_int(input_ids.shape[0]), c_int(prev_tokens.shape[0]),
                                           _stream())
    _check(st, "patch_token_ids")


# ---------------------------------------------------------------- norms

def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """y = x / sqrt(mean(x^2) + eps) * weight over the last dim; weight float32."""
    x = as_tensor(x)
    _need(x, "x")
    _need(weight, "weight", torch.float32, 1)
    h = x.shape[-1]
    if weight.shape[0] != h:
        raise KernelError(f"rms_norm: weight has {weight.shape[0]} elements, rows have {h}")
    out = torch.empty_like(x)
    rows = x.numel() // h if h else 0
    st = _lib("elementwise").dib_rms_norm(_ptr(x), _ptr(weight), _ptr(out), c_int(rows), c_int(h),
                                          c_float(eps), c_int(_dt(x, "x")), _stream())
    _check(st, "rms_norm", f"row width {h}")
    return out


def add_rms_norm(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, eps: float):
    """In place: residual += x (stored rounded); x = rms_norm(unrounded sum).
    Returns (x, residual).  ``x`` may be a ``SplitSum``; the norm is then written to
    a new tensor."""
    if isinstance(x, SplitSum):
        _need(residual, "residual", x.dtype, 2)
        _need(weight, "weight", torch.float32, 1)
        s_, rows, h = x.parts.shape
        if tuple(residual.shape) != (rows, h) or weight.shape[0] != h:
            raise KernelError(f"add_rms_norm: x {(rows, h)} vs residual {tuple(residual.shape)}, "
                              f"weight {weight.shape[0]}")
        if h % 4 == 0 and h <= (16384 if rows <= 128 else 4096):
            out = torch.empty(rows, h, dtype=x.dtype, device=x.device)
            st = _lib("elementwise").dib_add_rms_norm_split(
                _ptr(x.parts), c_int(s_), c_longlong(rows * h), _ptr(residual), _ptr(weight),
                _ptr(out), c_int(rows), c_int(h), c_float(eps), c_int(_DT[x.dtype]), _stream())
            _check(st, "add_rms_norm(split)", f"row width {h}")
            return out, residual
        x = x.tensor()
    _need(x, "x")
    _need(residual, "residual", x.dtype)
    _need(weight, "weight", torch.float32, 1)
    if x.shape != residual.shape:
        raise KernelError(f"add_rms_norm: x {tuple(x.shape)} vs residual {tuple(residual.shape)}")
    h = x.shape[-1]
    if weight.shape[0] != h:
        raise KernelError(f"add_rms_norm: weight has {weight.shape[0]} elements, rows have {h}")
    rows = x.numel() // h if h else 0
    st = _lib("elementwise").dib_add_rms_norm(_ptr(x), _ptr(residual), _ptr(weight), c_int(rows),
                                              c_int(h), c_float(eps), c_int(_dt(x, "x")), _stream())
    _check(st, "add_rms_norm", f"row width {h}")
    return x, residual


# ------------------------------------------------ q/k norm + rotary + cache

def qk_norm_rope_cache(qkv: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int,
                       q_norm_weight, k_norm_weight, eps: float, cos_sin, positions: torch.Tensor,
                       kv_cache, slot_mapping, page_size: int) -> torch.Tensor:
    """From the fused projection row [q heads | k heads | v heads] of each token:
    per-head RMSNorm of q and k (when a weight is given), rotate-half rotation by
    the token's position (when a table [max_pos, rotary_dim] = [cos | sin] is
    given), q to the returned tensor [T, Hq, D], k and v into the token's slot of
    the paged cache [pages, 2, Hkv, page_size, D] (when a cache is given;
    slot = page * page_size + offset, negative = skip)."""
    parts = None
    if isinstance(qkv, SplitSum):
        if head_dim in (64, 128, 256) and (cos_sin is None or cos_sin.shape[1] == head_dim):
            parts = qkv
        else:
            qkv = qkv.tensor()
    if parts is None:
        _need(qkv, "qkv", None, 2)
    t, got_width = qkv.shape
    act_dtype, device = qkv.dtype, qkv.device
    width = (num_heads + 2 * num_kv_heads) * head_dim
    if got_width != width:
        raise KernelError(f"qkv has width {got_width}, expected {width}")
    _need(positions, "positions", torch.int32, 1)
    for w, n in ((q_norm_weight, "q_norm_weight"), (k_norm_weight, "k_norm_weight")):
        if w is not None:
            _need(w, n, torch.float32, 1)
            if w.shape[0] != head_dim:
                raise KernelError(f"{n} has {w.shape[0]} elements, head_dim is {head_dim}")
    rotary_dim, max_pos = 0, 0
    if cos_sin is not None:
        _need(cos_sin, "cos_sin", torch.float32, 2)
        max_pos, rotary_dim = cos_sin.shape
    num_pages = 0
    if kv_cache is not None:
        _need(kv_cache, "kv_cache", act_dtype, 5)
        _need(slot_mapping, "slot_mapping", torch.int32, 1)
        if tuple(kv_cache.shape[1:]) != (2, num_kv_heads, page_size, head_dim):
            raise KernelError(f"kv_cache shape {tuple(kv_cache.shape)} does not match "
                              f"[pages, 2, {num_kv_heads}, {page_size}, {head_dim}]")
        num_pages = kv_cache.shape[0]
    q = torch.empty(t, num_heads, head_dim, dtype=act_dtype, device=device)
    if parts is not None:
        st = _lib("elementwise").dib_qk_norm_rope_cache_split(
            c_void_p(0), _ptr(parts.parts), c_int(parts.splits), c_longlong(t * width), _ptr(q),
            _ptr(kv_cache), _ptr(q_norm_weight), _ptr(k_norm_weight), c_float(eps), _ptr(cos_sin),
            c_int(rotary_dim), c_int(max_pos), _ptr(positions), _ptr(slot_mapping), c_int(t),
            c_int(num_heads), c_int(num_kv_heads), c_int(head_dim), c_int(page_size),
            c_longlong(num_pages), c_int(_DT[parts.dtype]), _stream())
        _check(st, "qk_norm_rope_cache(split)", f"head_dim {head_dim}")
        return q
    st = _lib("elementwise").dib_qk_norm_rope_cache(
        _ptr(qkv), _ptr(q), _ptr(kv_cache), _ptr(q_norm_weight), _ptr(k_norm_weight), c_float(eps),
        _ptr(cos_sin), c_int(rotary_dim), c_int(max_pos), _ptr(positions), _ptr(slot_mapping),
        c_int(t), c_int(num_heads), c_int(num_kv_heads), c_int(head_dim), c_int(page_size),
        c_longlong(num_pages), c_int(_dt(qkv, "qkv")), _stream())
    _check(st, "qk_norm_rope_cache", f"head_dim {head_dim}, rotary_dim {rotary_dim}")
    return q


def qkv_project(x: torch.Tensor, w_qkv: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int,
                q_norm_weight, k_norm_weight, eps: float, cos_sin, positions: torch.Tensor, kv_cache,
                slot_mapping, page_size: int) -> torch.Tensor:
    """The fused q/k/v projection of the step's tokens followed by ``qk_norm_rope_cache``: returns
    q [T, Hq, D], with k and v in the tokens' cache slots.  Many bfloat16 rows of heads of 128
    run as ONE kernel when the package's many-rows product is in use (``large_products`` "own"
    or "auto"): the product's epilogue norms, rotates and writes the cache, with the bits of
    the two kernels."""
    x = as_tensor(x)
    if x.dtype == torch.bfloat16 and x.is_cuda and head_dim == 128 and kv_cache is not None \
            and (cos_sin is None or cos_sin.shape[1] == head_dim):
        from . import gemm_bf16
        q = gemm_bf16.qkv_large(x, w_qkv, num_heads, num_kv_heads, q_norm_weight, k_norm_weight, eps,
                                cos_sin, positions, kv_cache, slot_mapping, page_size)
        if q is not None:
            return q
    return qk_norm_rope_cache(linear(x, w_qkv), num_heads, num_kv_heads, head_dim, q_norm_weight,
                              k_norm_weight, eps, cos_sin, positions, kv_cache, slot_mapping, page_size)


def reshape_and_cache(k: torch.Tensor, v: torch.Tensor, kv_cache: torch.Tensor,
                      slot_mapping: torch.Tensor) -> None:
    """k, v [T, Hkv, D] into their slots of the paged cache (negative slot: skip)."""
    _need(k, "k", None, 3)
    _need(v, "v", k.dtype, 3)
    _need(kv_cache, "kv_cache", k.dtype, 5)
    _need(slot_mapping, "slot_mapping", torch.int32, 1)
    t, hkv, d = k.shape
    if v.shape != k.shape or kv_cache.shape[1] != 2 or kv_cache.shape[2] != hkv or kv_cache.shape[4] != d:
        raise KernelError(f"reshape_and_cache: k {tuple(k.shape)}, v {tuple(v.shape)}, "
                          f"cache {tuple(kv_cache.shape)}")
    st = _lib("elementwise").dib_reshape_and_cache(
        _ptr(k), _ptr(v), _ptr(kv_cache), _ptr(slot_mapping), c_int(t), c_int(hkv), c_int(d),
        c_int(kv_cache.shape[3]), c_longlong(kv_cache.shape[0]), c_int(_dt(k, "k")), _stream())
    _check(st, "reshape_and_cache")


# ---------------------------------------------------------------- attention

def paged_attention(q: torch.Tensor, kv_cache: torch.Tensor, meta, scale: float,
                    window=None, defer: bool = False):
    """Causal attention of every token of the step over its sequence's keys in the
    paged cache.  q [T, Hq, D]; kv_cache [pages, 2, Hkv, page_size, D]; ``meta``
    is the step's attention metadata for this cache's group (``AttentionMeta``:
    block_table [B, max_blocks], token_seq [T], positions [T], cu_q_lens [B+1],
    seq_lens [B], host copies of the lengths, number of leading decode
    sequences).  A query at position p sees keys max(0, p-window+1) .. p.
    ``defer``: a step of one-token sequences only may come back as a ``SplitAttention``
    (its splits not yet merged) for the matrix product that follows to merge."""
    _need(q, "q", None, 3)
    _need(kv_cache, "kv_cache", q.dtype, 5)
    t, hq, d = q.shape
    _, two, hkv, page_size, d2 = kv_cache.shape
    if two != 2 or d2 != d or hq % hkv:
        raise KernelError(f"paged_attention: q {tuple(q.shape)} vs cache {tuple(kv_cache.shape)}")
    _need(meta.block_table, "block_table", torch.int32, 2)
    _need(meta.token_seq, "token_seq", torch.int32, 1)
    _need(meta.positions, "positions", torch.int32, 1)
    out = torch.empty_like(q)
    win = int(window) if window else 0
    if q.dtype == torch.bfloat16:
        from . import attention_bf16
        if attention_bf16.supports(hq, hkv, d, page_size):
            deferred = attention_bf16.run(q, out, kv_cache, meta, scale, win, defer)
            return deferred if deferred is not None else out
    st = _lib("attention_generic").dib_paged_attention_generic(
        _ptr(q), _ptr(out), _ptr(kv_cache), _ptr(meta.block_table), c_int(meta.block_table.shape[1]),
        _ptr(meta.token_seq), _ptr(meta.positions), c_int(t), c_int(hq), c_int(hkv), c_int(d),
        c_int(page_size), c_float(scale), c_int(win), c_int(_dt(q, "q")), _stream())
    _check(st, "paged_attention", f"head_dim {d} (at most 256), heads {hq}/{hkv}")
    return out


# ---------------------------------------------------------------- feed-forward

def silu_mul(gate_up: torch.Tensor) -> torch.Tensor:
    """[T, 2I] = [gate | up] -> silu(gate) * up, [T, I]."""
    if isinstance(gate_up, SplitSum):
        s_, t, two_i = gate_up.parts.shape
        if two_i % 8 == 0:
            out = torch.empty(t, two_i // 2, dtype=gate_up.dtype, device=gate_up.device)
            st = _lib("elementwise").dib_silu_mul_split(
                _ptr(gate_up.parts), c_int(s_), c_longlong(t * two_i), _ptr(out), c_int(t),
                c_int(two_i // 2), c_int(_DT[gate_up.dtype]), _stream())
            _check(st, "silu_mul(split)")
            return out
        gate_up = gate_up.tensor()
    _need(gate_up, "gate_up", None, 2)
    t, two_i = gate_up.shape
    if two_i % 2:
        raise KernelError(f"silu_mul: width {two_i} is odd")
    out = torch.empty(t, two_i // 2, dtype=gate_up.dtype, device=gate_up.device)
    st = _lib("elementwise").dib_silu_mul(_ptr(gate_up), _ptr(out), c_int(t), c_int(two_i // 2),
                                          c_int(_dt(gate_up, "gate_up")), _stream())
    _check(st, "silu_mul")
    return out


def gather_rows(x: torch.Tensor, index: torch.Tensor) -> torch.Tensor:
    """out[r] = x[index[r]]; index int32."""
    x = as_tensor(x)
    _need(x, "x", None, 2)
    _need(index, "index", torch.int32, 1)
    out = torch.empty(index.shape[0], x.shape[1], dtype=x.dtype, device=x.device)
    st = _lib("elementwise").dib_gather_rows(_ptr(x), _ptr(index), _ptr(out), c_int(index.shape[0]),
                                             c_int(x.shape[1]), c_int(x.shape[0]),
                                             c_int(_dt(x, "x")), _stream())
    _check(st, "gather_rows")
    return out


# ---------------------------------------------------------------- matrix product

def linear(x: torch.Tensor, weight: torch.Tensor, out_dtype=None) -> torch.Tensor:
    """y = x @ weight^T; x [M, K], weight [N, K] (checkpoint layout), no bias.

    float32: the package's own CUDA-core kernel (plain FMA, no TF32, fixed k
    order, so a row's bits do not depend on the batch).  bfloat16: float32
    accumulation on the tensor cores; ``out_dtype=torch.float32`` returns the
    accumulator unrounded (used for the logits).  With few rows and a split of k the
    bfloat16 product comes back as a ``SplitSum`` (see there)."""
    if isinstance(x, (GatedSplit, SplitAttention)) and weight.dtype == torch.bfloat16 \
            and tuple(x.shape)[1] == weight.shape[1]:
        from . import gemm_bf16
        y = gemm_bf16.linear_of_deferred(x, weight, out_dtype or torch.bfloat16)
        if y is not None:
            return y
    x = as_tensor(x)
    _need(x, "x", None, 2)
    _need(weight, "weight", x.dtype, 2)
    m, k = x.shape
    n, k2 = weight.shape
    if k != k2:
        raise KernelError(f"linear: x [{m}, {k}] against weight [{n}, {k2}]")
    if x.dtype == torch.float32:
        out = torch.empty(m, n, dtype=torch.float32, device=x.device)
        st = _lib("gemm_fp32").dib_gemm_fp32(_ptr(x), _ptr(weight), _ptr(out), c_int(m), c_int(n),
                                             c_int(k), _stream())
        _check(st, "linear(float32)", f"M={m} N={n} K={k}")
        return out
    if x.dtype != torch.bfloat16:
        raise KernelError(f"linear: dtype {x.dtype} is not supported")
    from . import gemm_bf16
    return gemm_bf16.linear(x, weight, out_dtype or torch.bfloat16)


def gated_linear(x: torch.Tensor, w_gate_up: torch.Tensor):
    """silu(x w_gate^T) * (x w_up^T), [M, I], for the concatenated weight
    [w_gate ; w_up] ([2I, K]).  With few bfloat16 rows the gate is applied in the matrix
    product's epilogue, or, when the product comes back as split-k partials, left to the
    reader (a ``GatedSplit``); otherwise this is ``silu_mul(linear(x, w_gate_up))``."""
    x = as_tensor(x)
    if x.dtype == torch.bfloat16 and x.is_cuda:
        _need(x, "x", None, 2)
        _need(w_gate_up, "w_gate_up", x.dtype, 2)
        if x.shape[1] != w_gate_up.shape[1]:
            raise KernelError(f"gated_linear: x {tuple(x.shape)} against weight {tuple(w_gate_up.shape)}")
        from . import gemm_bf16
        out = gemm_bf16.gated_linear(x, w_gate_up)
        if out is not None:
            return out
    y = linear(x, w_gate_up)
    if isinstance(y, SplitSum) and y.dtype == torch.bfloat16 and y.shape[1] % 16 == 0 \
            and y.shape[0] <= GATE_IN_PRODUCT_ROWS and y.shape[1] // 2 <= GATE_IN_PRODUCT_WIDTH:
        return GatedSplit(y)          # the gate is applied by the product that reads it
    return silu_mul(y)


# ---------------------------------------------------------------- sampling

def argmax(logits: torch.Tensor) -> torch.Tensor:
    """int32 [R]: index of the largest logit of each row, lowest index on ties."""
    _need(logits, "logits", torch.float32, 2)
    r, v = logits.shape
    out = torch.empty(r, dtype=torch.int32, device=logits.device)
    lib = _lib("sampling")
    if v > 8192 and r <= 65535:
        # wide rows: one block per chunk of the row, then a second tiny kernel
        chunks = -(-v // 4096)
        sv = torch.empty(r, chunks, dtype=torch.float32, device=logits.device)
        si = torch.empty(r, chunks, dtype=torch.int32, device=logits.device)
        st = lib.dib_argmax_two_stage(_ptr(logits), _ptr(sv), _ptr(si), _ptr(out), c_int(r), c_int(v),
                                      _stream())
        _check(st, "argmax", kernels=2)
        return out
    st = lib.dib_argmax(_ptr(logits), _ptr(out), c_int(r), c_int(v), _stream())
    _check(st, "argmax")
    return out


def gumbel_sample(logits: torch.Tensor, temperatures: torch.Tensor, seeds: torch.Tensor,
                  sample_positions: torch.Tensor, keep=None, top_ks=None, top_ps=None,
                  return_thresholds: bool = False):
    """int32 [R]: rows with temperature <= 0 take the argmax; the others the
    position-seeded Gumbel-max draw from softmax(logits / temperature), restricted
    to ids with keep != 0 when a mask (uint8 [R, V]) is given.  ``top_ks`` (int64 [R],
    <= 0: off) and ``top_ps`` (float32 [R], >= 1: off): top-k / top-p applied inside the
    kernels by a probability threshold found without a sort (``return_thresholds``: also
    the int32 bits of each row's smallest kept probability, 0 where nothing is dropped)."""
    _need(logits, "logits", torch.float32, 2)
    r, v = logits.shape
    _need(temperatures, "temperatures", torch.float32, 1)
    _need(seeds, "seeds", torch.int64, 1)
    _need(sample_positions, "sample_positions", torch.int64, 1)
    if not (temperatures.shape[0] == seeds.shape[0] == sample_positions.shape[0] == r):
        raise KernelError("gumbel_sample: per-row parameter lengths differ from the number of rows")
    if keep is not None:
        _need(keep, "keep", torch.uint8, 2)
        if tuple(keep.shape) != (r, v):
            raise KernelError(f"gumbel_sample: keep {tuple(keep.shape)} vs logits {(r, v)}")
    out = torch.empty(r, dtype=torch.int32, device=logits.device)
    lib = _lib("sampling")
    filtered = top_ks is not None or top_ps is not None
    if (v > 8192 or filtered) and r <= 65535:
        # a block per chunk of a row (normaliser, then scores), then the best chunk
        chunks = -(-v // 4096)
        sf = torch.empty(3, r, chunks, dtype=torch.float32, device=logits.device)
        si = torch.empty(r, chunks, dtype=torch.int32, device=logits.device)
        thresh = None
        if top_ks is not None or top_ps is not None:
            _need(top_ks, "top_ks", torch.int64, 1)
            _need(top_ps, "top_ps", torch.float32, 1)
            if top_ks.shape[0] != r or top_ps.shape[0] != r:
                raise KernelError("gumbel_sample: top_ks / top_ps lengths differ from the number of rows")
            thresh = torch.empty(r, dtype=torch.int32, device=logits.device)
            # histograms of the four radix passes: [4, r, 256] 64-bit masses, then 32-bit counts
            hist = torch.empty(4 * r * 256 * 3 // 2, dtype=torch.int64, device=logits.device)
        st = lib.dib_gumbel_sample_chunked(_ptr(logits), _ptr(temperatures), _ptr(seeds),
                                           _ptr(sample_positions), _ptr(keep), _ptr(top_ks),
                                           _ptr(top_ps), _ptr(thresh),
                                           _ptr(hist) if thresh is not None else c_void_p(0),
                                           _ptr(sf), _ptr(si), _ptr(out), c_int(r), c_int(v), _stream())
        _check(st, "gumbel_sample", kernels=3 if thresh is None else 7)
        return (out, thresh) if return_thresholds else out
    if filtered:
        raise KernelError("gumbel_sample: top_ks / top_ps with more than 65535 rows")
    st = lib.dib_gumbel_sample(_ptr(logits), _ptr(temperatures), _ptr(seeds), _ptr(sample_positions),
                               _ptr(keep), _ptr(out), c_int(r), c_int(v), _stream())
    _check(st, "gumbel_sample")
    return out
