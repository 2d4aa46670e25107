"""The allocation-free decode attention entry point, called through its exported
C symbol, against the regular entry point.

``dib_decode_attention_bf16_noalloc`` serves callers that cannot allocate device
memory when they need attention (a host that fixed its device memory at start-up,
a process whose memory is committed elsewhere, a plug-in running under an
allocator it may not re-enter): its scratch for the
per-split partial results is a fixed array inside the library, not a buffer from
the caller.  This file is collected last on purpose: a run that stops at the first
failure has then already run every other test.  It passes alone in a fresh process
and after the other tests.
"""

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

import pytest
import torch

from tests.attn_util import PagedCase

pytestmark = pytest.mark.gpu

MAX_FLOATS = 4 * 1024 * 1024      # DIB_NOALLOC_SCRATCH_FLOATS of the header


def _library():
    from deterministic_inference_b200.kernels import build
    lib = build.load_library("decode_attention_noalloc")
    fn = lib.dib_decode_attention_bf16_noalloc
    fn.restype = c_int
    need = lib.dib_decode_attention_noalloc_scratch_needed
    need.restype = c_longlong
    return fn, need


def _call(fn, q, out, cache, meta, scale, window, max_splits):
    hq, d = q.shape[1], q.shape[2]
    hkv, page = cache.shape[2], cache.shape[3]
    ptr = lambda t: c_void_p(t.data_ptr())
    return fn(ptr(q), ptr(out), ptr(cache), ptr(meta.block_table), c_int(meta.block_table.shape[1]),
              ptr(meta.seq_lens), c_int(q.shape[0]), c_int(max_splits), c_int(hq), c_int(hkv),
              c_int(d), c_int(page), c_float(scale), c_int(window),
              c_void_p(torch.cuda.current_stream().cuda_stream))


@pytest.mark.parametrize("hq,hkv,d,page,window", [(16, 8, 128, 16, 0), (6, 2, 32, 32, 40)])
def test_noalloc_entry_matches_regular_entry_twice(monkeypatch, hq, hkv, d, page, window):
    from deterministic_inference_b200.kernels import ops
    fn, need = _library()
    lens_a, lens_b = [1, 33, 257, 700, 128], [513, 2, 129]
    prev = None
    # two calls in a row: the second has other sizes and finds the first call's
    # partial results still in the shared scratch
    for lens, seed in ((lens_a, 31), (lens_b, 32)):
        case = PagedCase(lens, hkv, d, page, torch.bfloat16, seed=seed)
        meta = case.meta(list(range(len(lens))), [(n - 1, 1) for n in lens])
        g = torch.Generator().manual_seed(seed + 100)
        q = torch.randn(len(lens), hq, d, generator=g).to(device="cuda", dtype=torch.bfloat16)
        want = ops.paged_attention(q, case.cache, meta, d ** -0.5, window or None)
        # the regular entry point on the kernels this entry point launches (keys copied row
        # by row instead of page-wise by TMA)
        from deterministic_inference_b200.kernels import attention_bf16
        monkeypatch.setitem(attention_bf16.SWITCHES, "decode_tma", False)
        want_same = ops.paged_attention(q, case.cache, meta, d ** -0.5, window or None)
        monkeypatch.setitem(attention_bf16.SWITCHES, "decode_tma", True)
        out = torch.full_like(q, float("nan"))
        max_splits = -(-max(lens) // 128)
        assert need(c_int(len(lens)), c_int(max_splits), c_int(hq), c_int(d)) <= MAX_FLOATS
        rc = _call(fn, q, out, case.cache, meta, d ** -0.5, window, max_splits)
        assert rc == 0
        torch.cuda.synchronize()
        # against the default kernels: the tolerance of the bfloat16 kernel tests; against
        # the same kernels (same split size, same order): the same bits
        torch.testing.assert_close(out.float(), want.float(), atol=2e-2, rtol=2e-2)
        assert torch.equal(out, want_same)
        prev = out
    from deterministic_inference_b200.kernels import build
    lib = build.load_library("decode_attention_noalloc")
    assert lib.dib_decode_attention_noalloc_status() == 0


def test_noalloc_entry_refuses_what_does_not_fit():
    fn, need = _library()
    hq, hkv, d, page = 16, 8, 128, 16
    case = PagedCase([5], hkv, d, page, torch.bfloat16, seed=33)
    meta = case.meta([0], [(4, 1)])
    q = torch.zeros(1, hq, d, device="cuda", dtype=torch.bfloat16)
    out = torch.zeros_like(q)
    too_many_splits = MAX_FLOATS // (hq * (d + 1)) + 1
    assert need(c_int(1), c_int(too_many_splits), c_int(hq), c_int(d)) > MAX_FLOATS
    assert _call(fn, q, out, case.cache, meta, 1.0, 0, too_many_splits) == -2
    # a head size the kernels do not take is refused as well
    q2 = torch.zeros(1, 4, 24, device="cuda", dtype=torch.bfloat16)
    cache2 = torch.zeros(4, 2, 4, page, 24, device="cuda", dtype=torch.bfloat16)
    assert _call(fn, q2, torch.zeros_like(q2), cache2, meta, 1.0, 0, 1) == -2
    torch.cuda.synchronize()
