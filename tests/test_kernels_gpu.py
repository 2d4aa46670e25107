"""Each CUDA kernel alone against its plain PyTorch reference (tests/torch_kernels.py),
at sizes other than the engine's: odd widths, head sizes in steps of 16, group
ratios 1..8, shuffled pages, page and tile edges, window edges.  Patterned after
the reference's kernel tests (tests/test_01_triton_ops.py, test_02_flash_decode.py,
test_03_extend_attention.py, test_04_reshape_and_cache.py, test_07_sampler.py)."""

import pytest
import torch

from tests import torch_kernels as ref
from tests.attn_util import PagedCase, dense_reference

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype):
    # bfloat16: the reference's kernel tolerance (tests/conftest.py:35-37)
    return dict(atol=2e-2, rtol=2e-2) if dtype == torch.bfloat16 else dict(atol=2e-6, rtol=2e-6)


@pytest.fixture
def switches(monkeypatch):
    """Sets the kernels' measurement switches for one test and puts them back."""
    from ctypes import c_int
    from deterministic_inference_b200.kernels import attention_bf16, gemm_bf16
    from deterministic_inference_b200.kernels import ops as _ops

    class Switches:
        def attention(self, **kw):
            for k, v in kw.items():
                assert k in attention_bf16.SWITCHES, k
                monkeypatch.setitem(attention_bf16.SWITCHES, k, v)

        def chunk_tiles(self, n):
            monkeypatch.setattr(attention_bf16, "CHUNK_TILES", n)

        def gemm(self, cluster=-1, splits=-1):
            gemm_bf16.configure(int(cluster), int(splits))

        def gated(self, v):
            monkeypatch.setattr(gemm_bf16, "GATED", v)

        def merge_wide_from(self, n):
            _ops._lib("attention_bf16").dib_attention_bf16_set_merge_wide_from(c_int(n))

    yield Switches()
    gemm_bf16.configure(0, 0)
    _ops._lib("attention_bf16").dib_attention_bf16_set_merge_wide_from(c_int(49))


def ops():
    from deterministic_inference_b200.kernels import ops as o
    return o


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("h", [200, 201, 4096, 8])
def test_embedding(dtype, h):
    """Rows of a multiple of 16 bytes are copied 16 bytes a thread, others element by element;
    an id outside the table gives a row of zeros."""
    torch.manual_seed(0)
    table = torch.randn(1000, h, device="cuda").to(dtype)
    ids = torch.tensor([0, 999, 5, 5, 123, 998, 1], dtype=torch.int32, device="cuda")
    assert torch.equal(ops().embedding(ids, table), ref.embedding(ids, table))
    bad = torch.tensor([3, -1, 1000, 7], dtype=torch.int32, device="cuda")
    got = ops().embedding(bad, table)
    assert torch.equal(got[0], table[3]) and torch.equal(got[3], table[7])
    assert float(got[1].abs().sum()) == 0.0 and float(got[2].abs().sum()) == 0.0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,h", [(1, 1024), (7, 5120), (33, 200), (128, 96), (3, 12288),
                                    (200, 5120), (70, 8192), (65, 4100), (2, 16384), (100, 20000)])
def test_rms_norm(dtype, rows, h):
    torch.manual_seed(1)
    x = torch.randn(rows, h, device="cuda").to(dtype)
    w = torch.randn(h, device="cuda")
    got = ops().rms_norm(x, w, 1e-5)
    want = ref._rms(x.float(), w, 1e-5)
    torch.testing.assert_close(got.float(), want, **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,h", [(1, 1024), (9, 4096), (33, 200), (200, 5120), (66, 8192),
                                    (3, 16384), (80, 12288)])
def test_add_rms_norm(dtype, rows, h):
    torch.manual_seed(2)
    x = torch.randn(rows, h, device="cuda").to(dtype)
    r = torch.randn(rows, h, device="cuda").to(dtype)
    w = torch.randn(h, device="cuda")
    s = x.float() + r.float()
    gx, gr = ops().add_rms_norm(x.clone(), r.clone(), w, 1e-6)
    torch.testing.assert_close(gr.float(), s.to(dtype).float(), atol=0, rtol=0)   # stored rounded
    torch.testing.assert_close(gx.float(), ref._rms(s, w, 1e-6), **tol(dtype))    # norm of unrounded sum


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hq,hkv,d,rot,norm,t", [
    (16, 8, 128, 128, True, 37), (6, 2, 32, 32, True, 37), (5, 5, 48, 48, True, 37), (4, 1, 80, 32, False, 37),
    (8, 1, 16, 16, True, 37), (3, 3, 64, 0, True, 37), (7, 7, 256, 256, True, 37),
    # many rows of 128: the kernel with eight lanes per row (odd head counts, rows that end a group)
    (16, 8, 128, 128, True, 301), (5, 1, 128, 128, True, 333), (12, 4, 128, 128, False, 200),
    (16, 8, 128, 0, True, 129)])
def test_qk_norm_rope_cache(dtype, hq, hkv, d, rot, norm, t):
    torch.manual_seed(3)
    page, max_pos = 16, 300
    pages = -(-t // page) + 3
    qkv = torch.randn(t, (hq + 2 * hkv) * d, device="cuda").to(dtype)
    qw = torch.randn(d, device="cuda") if norm else None
    kw = torch.randn(d, device="cuda") if norm else None
    table = None
    if rot:
        half = rot // 2
        inv = 1.0 / (1e4 ** (torch.arange(half, dtype=torch.float32, device="cuda") / half))
        f = torch.outer(torch.arange(max_pos, dtype=torch.float32, device="cuda"), inv)
        table = torch.cat([f.cos(), f.sin()], -1).contiguous()
    pos = torch.randint(0, max_pos, (t,), device="cuda", dtype=torch.int32)
    slots = (torch.randperm((pages - 1) * page, device="cuda")[:t] + page).to(torch.int32)
    slots[5] = -1                                   # skipped token
    c1 = torch.zeros(pages, 2, hkv, page, d, device="cuda", dtype=dtype)
    c2 = c1.clone()
    q1 = ops().qk_norm_rope_cache(qkv, hq, hkv, d, qw, kw, 1e-6, table, pos, c1, slots, page)
    q2 = ref.qk_norm_rope_cache(qkv, hq, hkv, d, qw, kw, 1e-6, table, pos, c2, slots, page)
    torch.testing.assert_close(q1.float(), q2.float(), **tol(dtype))
    torch.testing.assert_close(c1.float(), c2.float(), **tol(dtype))
    assert torch.equal(c1[0], torch.zeros_like(c1[0]))      # page 0 untouched
    # without a cache nothing is written and q is the same
    q3 = ops().qk_norm_rope_cache(qkv, hq, hkv, d, qw, kw, 1e-6, table, pos, None, None, page)
    assert torch.equal(q1, q3)


@pytest.mark.parametrize("dtype", DTYPES)
def test_reshape_and_cache_round_trip(dtype):
    torch.manual_seed(4)
    t, hkv, d, page, pages = 50, 3, 48, 8, 20
    k = torch.randn(t, hkv, d, device="cuda").to(dtype)
    v = torch.randn(t, hkv, d, device="cuda").to(dtype)
    slots = (torch.randperm((pages - 1) * page, device="cuda")[:t] + page).to(torch.int32)
    slots[0] = -1
    cache = torch.zeros(pages, 2, hkv, page, d, device="cuda", dtype=dtype)
    ops().reshape_and_cache(k, v, cache, slots)
    for i in range(1, t):
        p, o = int(slots[i]) // page, int(slots[i]) % page
        assert torch.equal(cache[p, 0, :, o], k[i]) and torch.equal(cache[p, 1, :, o], v[i])
    assert cache.float().abs().sum() == (k[1:].float().abs().sum() + v[1:].float().abs().sum())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("t,i", [(1, 3072), (5, 160), (64, 25600), (3, 7)])
def test_silu_mul(dtype, t, i):
    torch.manual_seed(5)
    gu = (3 * torch.randn(t, 2 * i, device="cuda")).to(dtype)
    g, u = gu[:, :i].float(), gu[:, i:].float()
    torch.testing.assert_close(ops().silu_mul(gu).float(), g * torch.sigmoid(g) * u, **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("h", [200, 203, 4096])
def test_gather_rows(dtype, h):
    x = torch.randn(40, h, device="cuda").to(dtype)
    idx = torch.tensor([39, 0, 7, 7], dtype=torch.int32, device="cuda")
    assert torch.equal(ops().gather_rows(x, idx), x[idx.long()])


@pytest.mark.parametrize("m,n,k", [(1, 151, 97), (33, 200, 130), (70, 64, 64), (2, 1000, 1024),
                                   (257, 96, 160)])
def test_linear_fp32_is_true_fp32(m, n, k):
    torch.manual_seed(6)
    x = torch.randn(m, k, device="cuda")
    w = torch.randn(n, k, device="cuda")
    got = ops().linear(x, w)
    want = (x.double() @ w.double().T)
    # float32 FMA accumulation: error ~ k * 2^-24 * |terms|; TF32 would be ~1e-3
    torch.testing.assert_close(got.double(), want, atol=2e-5 * (k ** 0.5), rtol=1e-5)


def test_linear_fp32_row_does_not_depend_on_batch():
    """A row gives the same bits alone and among 333 rows (the reference checks its
    batch-invariant product the same way, tests/test_10_batch_invariant.py:32-43)."""
    torch.manual_seed(7)
    x = torch.randn(333, 200, device="cuda")
    w = torch.randn(150, 200, device="cuda")
    full = ops().linear(x, w)
    for r in (0, 63, 64, 332):
        assert torch.equal(ops().linear(x[r:r + 1].contiguous(), w)[0], full[r])


@pytest.mark.parametrize("m,n,k", [
    (1, 4096, 1024), (8, 1024, 3072), (8, 1024, 2048), (8, 6144, 1024), (64, 200, 136),
    (17, 130, 72), (128, 256, 64), (33, 100, 8), (5, 151936, 1024), (100, 3000, 520),
    (129, 152, 96), (300, 152, 96), (2048, 512, 256)])
@pytest.mark.parametrize("cluster", ["1", "0"])
def test_linear_bf16(m, n, k, cluster, switches):
    """Few rows (up to ``gemm_bf16.MAX_ROWS``) run the package's swap-AB tcgen05 kernel (tails
    in N and K, split k), more rows the library or the many-rows kernel.  A split of k is
    added up by the tile's cluster of CTAs (a finished tensor comes back) or left as partial
    products.  With the library switched off the few-rows kernel takes every row count (one
    to many token tiles): the sizes above the line run on it too."""
    from deterministic_inference_b200.kernels import gemm_bf16
    switches.gemm(cluster=cluster)
    torch.manual_seed(8)
    x = torch.randn(m, k, device="cuda").to(torch.bfloat16)
    w = (0.05 * torch.randn(n, k, device="cuda")).to(torch.bfloat16)
    want = x.float() @ w.float().T
    modes = [True] if m <= gemm_bf16.MAX_ROWS else [True, False]
    try:
        for library in modes:
            gemm_bf16.set_library_products(library)
            got = ops().linear(x, w)
            assert isinstance(got, ops().SplitSum) == (cluster == "0" and m <= gemm_bf16.MAX_ROWS
                                                       and gemm_bf16.plan(m, n, k, x.device)[2] > 1)
            torch.testing.assert_close(ops().as_tensor(got).float(), want, atol=2e-2, rtol=2e-2)
            got32 = ops().as_tensor(ops().linear(x, w, out_dtype=torch.float32))
            assert got32.dtype == torch.float32
            torch.testing.assert_close(got32, want, atol=1e-3, rtol=1e-3)
    finally:
        gemm_bf16.set_library_products(True)
    assert gemm_bf16.status() == 0


def test_linear_bf16_row_does_not_depend_on_batch():
    """The k order and the split of k depend on N and K only: a row alone and among
    100 rows gives the same bits; and a second launch finds its counters reset."""
    torch.manual_seed(9)
    x = torch.randn(100, 2048, device="cuda").to(torch.bfloat16)
    w = (0.05 * torch.randn(1024, 2048, device="cuda")).to(torch.bfloat16)
    lin = lambda a: ops().as_tensor(ops().linear(a, w))
    full = lin(x)
    for r in (0, 15, 16, 99):
        assert torch.equal(lin(x[r:r + 1].contiguous())[0], full[r])
    assert torch.equal(lin(x), full)


@pytest.mark.parametrize("m,i,k", [(1, 3072, 1024), (8, 128, 72), (40, 192, 520), (100, 64, 64),
                                   (200, 128, 96), (8, 100, 64)])
def test_gated_linear(m, i, k, switches):
    """silu(x Wg^T) * (x Wu^T) with the gate in the product's epilogue (few rows, I a
    multiple of 64) or as two kernels; both against the formula with the two products
    rounded to bfloat16 as stored."""
    switches.gated("1")      # also the small shapes take the epilogue
    torch.manual_seed(12)
    x = torch.randn(m, k, device="cuda").to(torch.bfloat16)
    w = (0.08 * torch.randn(2 * i, k, device="cuda")).to(torch.bfloat16)
    y = (x.float() @ w.float().T).to(torch.bfloat16).float()
    g, u = y[:, :i], y[:, i:]
    want = g * torch.sigmoid(g) * u
    got = ops().gated_linear(x, w)
    assert got.shape == (m, i) and got.dtype == torch.bfloat16
    torch.testing.assert_close(got.float(), want, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("m,n,k,splits", [(8, 1024, 2048, 8), (1, 4096, 1024, 4), (64, 1024, 3072, 6),
                                          (128, 300, 520, 3), (17, 6144, 1024, 2), (33, 200, 1024, 7)])
def test_cluster_sum_of_a_split_gives_the_bits_of_the_partials(m, n, k, splits, switches):
    """The same split of k (forced), once added up by the tile's cluster through
    distributed shared memory, once left as partial products that a reader adds in split
    order: the same bits, in bfloat16 and float32 outputs; and the gate after a cluster's
    sum gives what the gate kernel gives on the partials."""
    from deterministic_inference_b200.kernels import gemm_bf16
    switches.gemm(splits=splits)
    torch.manual_seed(14)
    x = torch.randn(m, k, device="cuda").to(torch.bfloat16)
    w = (0.05 * torch.randn(n, k, device="cuda")).to(torch.bfloat16)
    outs = {}
    gemm_bf16.set_library_products(False)      # the few-rows kernel whatever the row count
    try:
        for cluster in ("1", "0"):
            switches.gemm(cluster=cluster)
            y = ops().linear(x, w)
            assert isinstance(y, ops().SplitSum) == (cluster == "0")
            outs[cluster] = (ops().as_tensor(y), ops().as_tensor(ops().linear(x, w, out_dtype=torch.float32)))
        assert torch.equal(outs["1"][0], outs["0"][0]) and torch.equal(outs["1"][1], outs["0"][1])
        if n % 128 == 0:
            gated = {}
            for cluster in ("1", "0"):
                switches.gemm(cluster=cluster)
                switches.gated("1" if cluster == "1" else "0")
                gated[cluster] = ops().as_tensor(ops().gated_linear(x, w))
            assert torch.equal(gated["1"], gated["0"])
    finally:
        gemm_bf16.set_library_products(True)


@pytest.mark.parametrize("m", [1, 8, 50])
def test_readers_of_split_k_partials(m):
    """The kernels that take a projection output as split-k partials give what they
    give on the summed tensor."""
    o = ops()
    torch.manual_seed(10)
    h, i, hq, hkv, d = 1024, 3072, 16, 8, 128
    x = torch.randn(m, h, device="cuda").to(torch.bfloat16)
    res = torch.randn(m, h, device="cuda").to(torch.bfloat16)
    wn = torch.randn(h, device="cuda")
    mk = lambda n, k: (0.05 * torch.randn(n, k, device="cuda")).to(torch.bfloat16)
    # residual-add + norm reading the output projection
    a = torch.randn(m, 2048, device="cuda").to(torch.bfloat16)
    wo = mk(h, 2048)
    y = o.linear(a, wo)
    assert isinstance(y, o.SplitSum)
    got, r1 = o.add_rms_norm(y, res.clone(), wn, 1e-6)
    want, r2 = o.add_rms_norm(y.tensor(), res.clone(), wn, 1e-6)
    assert torch.equal(got, want) and torch.equal(r1, r2)
    # SiLU gate reading gate_up
    gu = o.linear(x, mk(2 * i, h))
    assert isinstance(gu, o.SplitSum)
    assert torch.equal(o.silu_mul(gu), o.silu_mul(gu.tensor()))
    # q/k norm + rotation + cache write reading qkv
    qkv = o.linear(x, mk((hq + 2 * hkv) * d, h))
    assert isinstance(qkv, o.SplitSum)
    half = d // 2
    inv = 1.0 / (1e6 ** (torch.arange(half, dtype=torch.float32, device="cuda") / half))
    f = torch.outer(torch.arange(64, dtype=torch.float32, device="cuda"), inv)
    table = torch.cat([f.cos(), f.sin()], -1).contiguous()
    pos = torch.randint(0, 64, (m,), device="cuda", dtype=torch.int32)
    slots = (torch.randperm(5 * 16, device="cuda")[:m] + 16).to(torch.int32)
    c1 = torch.zeros(7, 2, hkv, 16, d, device="cuda", dtype=torch.bfloat16)
    c2 = c1.clone()
    qn, kn = torch.randn(d, device="cuda"), torch.randn(d, device="cuda")
    q1 = o.qk_norm_rope_cache(qkv, hq, hkv, d, qn, kn, 1e-6, table, pos, c1, slots, 16)
    q2 = o.qk_norm_rope_cache(qkv.tensor(), hq, hkv, d, qn, kn, 1e-6, table, pos, c2, slots, 16)
    assert torch.equal(q1, q2) and torch.equal(c1, c2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,h,splits", [(3, 5120, 2), (100, 5120, 3), (128, 8192, 2), (5, 16384, 4),
                                           (128, 20000, 2), (7, 1028, 5)])
def test_add_rms_norm_of_partials_wide_rows(dtype, rows, h, splits):
    """Residual-add + norm reading split-k partials at row widths beyond what one
    pass of a block covers (also the widths that take the summed-tensor route)."""
    o = ops()
    torch.manual_seed(rows + h)
    parts = torch.randn(splits, rows, h, device="cuda")
    res = torch.randn(rows, h, device="cuda").to(dtype)
    w = torch.randn(h, device="cuda")
    got, r1 = o.add_rms_norm(o.SplitSum(parts, dtype), res.clone(), w, 1e-5)
    acc = parts[0].clone()
    for i in range(1, splits):
        acc += parts[i]
    x = acc.to(dtype)
    want, r2 = ref.add_rms_norm(x.clone(), res.clone(), w, 1e-5)
    tol = dict(atol=1e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(r1.float(), r2.float(), **tol)
    torch.testing.assert_close(got.float(), want.float(), **tol)


# ------------------------------------------------------------------ attention

ATTN_SHAPES = [(16, 8, 128, 16), (6, 2, 32, 32), (5, 5, 48, 16), (8, 1, 64, 8), (4, 4, 16, 64),
               (64, 8, 128, 16), (2, 2, 256, 16)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hq,hkv,d,page", ATTN_SHAPES)
def test_paged_attention_mixed_batch(dtype, hq, hkv, d, page):
    """Decode tokens beside prompt portions with cached prefixes, shuffled pages;
    lengths at page and tile edges (tests/test_02_flash_decode.py:61-71,
    tests/test_03_extend_attention.py:56-72 of the reference)."""
    lens = [1, 33, 257, 64, 100, 31]
    case = PagedCase(lens, hkv, d, page, dtype, seed=11)
    # seq: (first new position, new tokens)
    cuts = [(0, 1), (32, 1), (256, 1), (0, 64), (37, 63), (29, 2)]
    seqs = list(range(len(lens)))
    meta = case.meta(seqs, cuts)
    g = torch.Generator().manual_seed(12)
    t = sum(n for _, n in cuts)
    q = torch.randn(t, hq, d, generator=g).to(device="cuda", dtype=dtype)
    got = ops().paged_attention(q, case.cache, meta, d ** -0.5)
    off = 0
    for s, (start, n) in zip(seqs, cuts):
        want = dense_reference(q[off:off + n], case.k[s], case.v[s], d ** -0.5,
                               list(range(start, start + n)))
        torch.testing.assert_close(got[off:off + n].float(), want, **tol(dtype))
        off += n


@pytest.mark.parametrize("hq,hkv,d,page,window", [(16, 8, 128, 16, None), (8, 2, 128, 8, 300), (64, 8, 128, 128, None),
                                                  (4, 1, 64, 32, None), (6, 3, 64, 16, 129), (32, 8, 128, 64, 1000)])
def test_decode_attention_pipelined_walk_gives_the_same_bits(switches, hq, hkv, d, page, window):
    """The decode kernel that walks many splits per CTA with its copies pipelined gives,
    bit for bit, what the one-split-per-CTA kernel gives (each split is computed alike),
    with enough splits that every CTA reuses its stages several times, ragged lengths at
    split and page edges, and windows that cut splits off the front; both agree with the
    dense reference."""
    g = torch.Generator().manual_seed(5)
    n_seq = 24 * max(1, 8 // hkv)
    lens = torch.randint(1, 1400, (n_seq,), generator=g).tolist()
    lens[:6] = [1, 128, 129, 1280, 127, 1399]
    case = PagedCase(lens, hkv, d, page, torch.bfloat16, seed=21)
    seqs = list(range(n_seq))
    meta = case.meta(seqs, [(n - 1, 1) for n in lens])
    q = torch.randn(n_seq, hq, d, generator=g).to(device="cuda", dtype=torch.bfloat16)
    outs = {}
    for mode in ("0", "1"):
        switches.attention(decode_pipe=int(mode))
        outs[mode] = ops().paged_attention(q, case.cache, meta, d ** -0.5, window).clone()
    assert ops()._lib("attention_bf16").dib_attention_bf16_status() == 0
    assert torch.equal(outs["0"], outs["1"])
    for s in (0, 1, 2, 3, 5, n_seq - 1):
        want = dense_reference(q[s:s + 1], case.k[s], case.v[s], d ** -0.5, [lens[s] - 1], window)
        torch.testing.assert_close(outs["1"][s:s + 1].float(), want, **tol(torch.bfloat16))


@pytest.mark.parametrize("hq,hkv,d,page,window", [(16, 8, 128, 16, None), (8, 2, 128, 32, 2500), (6, 3, 64, 16, None)])
def test_decode_attention_long_sequences_beside_short_ones(switches, hq, hkv, d, page, window):
    """Sequences of more than 16 splits of 128 keys: their splits are added chunk by chunk
    (16 splits), by one thread per dimension or by a group of threads per chunk, with the
    same bits; a short sequence beside them keeps the bits it has alone (the order of its
    sum depends on its own length only), both launch forms of stage 1 agree in every bit,
    and all agree with the dense reference."""
    lens = [5000, 300, 2049, 2048, 129, 4097]
    case = PagedCase(lens, hkv, d, page, torch.bfloat16, seed=61)
    g = torch.Generator().manual_seed(62)
    q = torch.randn(len(lens), hq, d, generator=g).to(device="cuda", dtype=torch.bfloat16)
    seqs = list(range(len(lens)))
    outs = {}
    for mode in ("0", "1"):
        switches.attention(decode_pipe=int(mode))
        outs[mode] = ops().paged_attention(q, case.cache, case.meta(seqs, [(n - 1, 1) for n in lens]),
                                           d ** -0.5, window).clone()
    assert ops()._lib("attention_bf16").dib_attention_bf16_status() == 0
    assert torch.equal(outs["0"], outs["1"])
    switches.attention(decode_pipe=2)
    for wide_from in (17, 100000):
        switches.merge_wide_from(wide_from)
        got = ops().paged_attention(q, case.cache, case.meta(seqs, [(n - 1, 1) for n in lens]),
                                    d ** -0.5, window)
        assert torch.equal(got, outs["0"]), wide_from
    switches.merge_wide_from(49)
    for s_ in seqs:
        want = dense_reference(q[s_:s_ + 1], case.k[s_], case.v[s_], d ** -0.5, [lens[s_] - 1], window)
        torch.testing.assert_close(outs["0"][s_:s_ + 1].float(), want, **tol(torch.bfloat16))
    # the short ones alone (at most 16 splits in the batch: the other merge kernel)
    short = [1, 3, 4]
    alone = ops().paged_attention(q[short].contiguous(), case.cache,
                                  case.meta(short, [(lens[i] - 1, 1) for i in short]), d ** -0.5, window)
    assert torch.equal(alone, outs["0"][short])


@pytest.mark.parametrize("tma", ["0", "1"])
def test_decode_attention_reads_its_partial_results_after_they_are_written(switches, tma):
    """The kernel that merges the splits starts beside the kernel that writes them
    (programmatic dependent launch) and must not read a partial result before its wait:
    the scratch is filled with NaN, huge values and plain numbers before each call, and
    every call gives the bits of the first."""
    switches.attention(decode_tma=tma == "1")
    hq, hkv, d, page = 16, 8, 128, 16
    lens = [513, 2, 129, 1, 33, 257, 700, 128]
    case = PagedCase(lens, hkv, d, page, torch.bfloat16, seed=3)
    meta = case.meta(list(range(len(lens))), [(n - 1, 1) for n in lens])
    g = torch.Generator().manual_seed(4)
    q = torch.randn(len(lens), hq, d, generator=g).to(device="cuda", dtype=torch.bfloat16)
    ref = ops().paged_attention(q, case.cache, meta, d ** -0.5, None).clone()
    scratch = [v for k, v in meta.scratch.items() if k[0] == "decode_ws"]
    assert len(scratch) == 1
    for rep in range(4):
        for fill in (float("nan"), 1e30, -1e30, 0.0, 123.0):
            for w in scratch[0]:
                w.fill_(fill)
            out = ops().paged_attention(q, case.cache, meta, d ** -0.5, None)
            assert torch.equal(out, ref), (rep, fill)
    for s_ in (0, 1, 6):
        want = dense_reference(q[s_:s_ + 1], case.k[s_], case.v[s_], d ** -0.5, [lens[s_] - 1], None)
        torch.testing.assert_close(ref[s_:s_ + 1].float(), want, **tol(torch.bfloat16))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [1, 7, 16, 24, 33, 500])
def test_paged_attention_window_edge(dtype, window):
    """One key far outside and one just inside the window carry huge values: the
    output shows at once whether the edge is off by one."""
    hq, hkv, d, page = 4, 2, 32, 16
    n = 90
    g = torch.Generator().manual_seed(13)
    k = [torch.randn(n, hkv, d, generator=g).to(device="cuda", dtype=dtype)]
    v = [torch.randn(n, hkv, d, generator=g).to(device="cuda", dtype=dtype)]
    case = PagedCase([n], hkv, d, page, dtype, seed=14, k=k, v=v)
    q = torch.randn(n - 40, hq, d, generator=g).to(device="cuda", dtype=dtype)
    meta = case.meta([0], [(40, n - 40)])
    got = ops().paged_attention(q, case.cache, meta, d ** -0.5, window)
    want = dense_reference(q, k[0], v[0], d ** -0.5, list(range(40, n)), window)
    torch.testing.assert_close(got.float(), want, **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
def test_paged_attention_far_key_stands_out(dtype):
    """Among 700 keys one early key matches the query strongly: the output must be
    that key's value (a kernel that skips a page or a tile would miss it)."""
    hq, hkv, d, page, n = 4, 2, 64, 16, 700
    g = torch.Generator().manual_seed(15)
    for far in (0, 15, 16, 255, 256, 300, 698):
        k = 0.1 * torch.randn(n, hkv, d, generator=g)
        v = torch.randn(n, hkv, d, generator=g)
        q = 0.1 * torch.randn(1, hq, d, generator=g)
        direction = torch.randn(d, generator=g)
        direction /= direction.norm()
        k[far] += 30 * direction
        q += 30 * direction
        case = PagedCase([n], hkv, d, page, dtype, seed=16,
                         k=[k.to(device="cuda", dtype=dtype)], v=[v.to(device="cuda", dtype=dtype)])
        qd = q.to(device="cuda", dtype=dtype)
        got = ops().paged_attention(qd, case.cache, case.meta([0], [(n - 1, 1)]), 1.0)
        for h in range(hq):
            torch.testing.assert_close(got[0, h].float(), case.v[0][far, h // 2].float(),
                                       atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("mode", ["0", "1", "2", "2-pairs", "2-alone"])
@pytest.mark.parametrize("hq,hkv,page,window", [(16, 8, 16, None), (32, 8, 16, 300), (8, 8, 32, None),
                                                (16, 1, 128, 200), (64, 8, 8, None)])
def test_prefill_attention_head_size_128_kernels(switches, mode, hq, hkv, page, window):
    """The three bfloat16 prompt kernels for heads of 128 (mma.sync; tcgen05 with one
    query tile per CTA; tcgen05 with two, as the step's size decides, with tiles paired
    from both ends of a prompt, and with a CTA for every tile) on prompts that span many
    key tiles: whole, behind a cached prefix, ending one token after a tile edge; group
    sizes 1 to 16."""
    switches.attention(prefill_tc=mode[0])
    if len(mode) > 1:
        switches.attention(prefill_pair="1" if mode.endswith("pairs") else "0")
    d = 128
    lens = [700, 300, 129, 257]
    cuts = [(0, 700), (100, 200), (1, 128), (0, 257)]
    case = PagedCase(lens, hkv, d, page, torch.bfloat16, seed=41)
    g = torch.Generator().manual_seed(42)
    q = torch.randn(sum(n for _, n in cuts), hq, d, generator=g).to(device="cuda", dtype=torch.bfloat16)
    got = ops().paged_attention(q, case.cache, case.meta([0, 1, 2, 3], cuts), d ** -0.5, window)
    assert ops()._lib("attention_prefill_tc").dib_attention_prefill_tc_status() == 0
    off = 0
    for s_, (start, n) in enumerate(cuts):
        want = dense_reference(q[off:off + n], case.k[s_], case.v[s_], d ** -0.5,
                               list(range(start, start + n)), window)
        torch.testing.assert_close(got[off:off + n].float(), want, **tol(torch.bfloat16))
        off += n


@pytest.mark.parametrize("hq,hkv,window", [(4, 2, None), (8, 2, 1100), (2, 2, None)])
def test_prefill_attention_key_range_shared_by_several_ctas(switches, hq, hkv, window):
    """Key ranges are cut at fixed multiples of a chunk (here 1,024 keys instead of the
    product's 4,096, so that small cases cross cuts); several CTAs take the chunks of a
    query tile and a merge adds their partial results: a whole prompt of three chunks, a
    portion behind a prefix whose range starts inside a chunk, a short sequence that one
    chunk finishes, and a decode token beside them; against the dense reference and
    against the run with one chunk."""
    d, page = 128, 16
    lens = [5, 2500, 1500, 200]
    cuts = [(4, 1), (0, 2500), (1100, 400), (0, 200)]
    case = PagedCase(lens, hkv, d, page, torch.bfloat16, seed=51)
    g = torch.Generator().manual_seed(52)
    q = torch.randn(sum(n for _, n in cuts), hq, d, generator=g).to(device="cuda", dtype=torch.bfloat16)
    outs = {}
    for chunk in (8, 32):
        switches.chunk_tiles(chunk)
        outs[chunk] = ops().paged_attention(q, case.cache, case.meta([0, 1, 2, 3], cuts), d ** -0.5, window)
    assert ops()._lib("attention_prefill_tc").dib_attention_prefill_tc_status() == 0
    torch.testing.assert_close(outs[8].float(), outs[32].float(), **tol(torch.bfloat16))
    off = 0
    for s_, (start, n) in enumerate(cuts):
        rows = list(range(0, n, 7)) + [n - 1]          # every 7th position, and the last
        want = dense_reference(q[off:off + n][rows], case.k[s_], case.v[s_], d ** -0.5,
                               [start + r for r in rows], window)
        torch.testing.assert_close(outs[8][off:off + n][rows].float(), want, **tol(torch.bfloat16))
        off += n


@pytest.mark.parametrize("chunk", [8, 32])
@pytest.mark.parametrize("hq,hkv,window", [(4, 2, None), (8, 1, 1500)])
def test_prefill_attention_bits_depend_on_the_position_alone(switches, chunk, hq, hkv, window):
    """The same query rows (positions 2,000..2,511 of a sequence) give the same bits
    whether their step holds them alone behind a prefix, the whole prompt, a longer
    portion, or other sequences beside them (longer and shorter ones, prompt portions and
    decode tokens): the key tiles and the chunk cuts are anchored at position 0, and how
    query tiles are paired or spread over CTAs is the only thing the step decides.  With
    chunks of 1,024 keys (several per row, merged) and of 4,096 (one)."""
    switches.chunk_tiles(chunk)
    d, page = 128, 16
    lens = [2512, 5000, 300, 77]
    case = PagedCase(lens, hkv, d, page, torch.bfloat16, seed=71)
    g = torch.Generator().manual_seed(72)
    q_all = torch.randn(2512, hq, d, generator=g).to(device="cuda", dtype=torch.bfloat16)
    q_other = torch.randn(1024, hq, d, generator=g).to(device="cuda", dtype=torch.bfloat16)
    scale = d ** -0.5

    def run(entries):        # entries: [(sequence, start, count, queries)]
        qs = torch.cat([e[3] for e in entries])
        meta = case.meta([e[0] for e in entries], [(e[1], e[2]) for e in entries])
        out = ops().paged_attention(qs, case.cache, meta, scale, window)
        res, off = {}, 0
        for e in entries:
            res[e[0]] = out[off:off + e[2]]
            off += e[2]
        return res

    alone = run([(0, 2000, 512, q_all[2000:2512])])[0]
    whole = run([(0, 0, 2512, q_all)])[0][2000:]
    longer = run([(0, 1990, 522, q_all[1990:2512])])[0][10:]
    # decode tokens first (the batch order of a step), then portions of other sequences
    mixed = run([(2, 299, 1, q_other[:1]), (3, 76, 1, q_other[1:2]),
                 (0, 2000, 512, q_all[2000:2512]), (1, 4200, 800, q_other[2:802])])[0]
    assert torch.equal(alone, whole)
    assert torch.equal(alone, longer)
    assert torch.equal(alone, mixed)
    want = dense_reference(q_all[2000:2512:37], case.k[0], case.v[0], scale, list(range(2000, 2512, 37)), window)
    torch.testing.assert_close(alone[::37].float(), want, **tol(torch.bfloat16))


@pytest.mark.parametrize("mode", ["1", "2"])
def test_prefill_attention_far_key_stands_out(switches, mode):
    """In a 700-token prompt one key matches every query strongly: each position at or
    after it must return that key's value, whichever key tile and query tile it is in."""
    switches.attention(prefill_tc=mode)
    hq, hkv, d, page, n = 4, 2, 128, 16, 700
    g = torch.Generator().manual_seed(43)
    for far in (0, 127, 128, 383, 500):
        k = 0.1 * torch.randn(n, hkv, d, generator=g)
        v = torch.randn(n, hkv, d, generator=g)
        q = 0.1 * torch.randn(n, hq, d, generator=g)
        direction = torch.randn(d, generator=g)
        direction /= direction.norm()
        k[far] += 30 * direction
        q += 30 * direction
        case = PagedCase([n], hkv, d, page, torch.bfloat16, seed=44,
                         k=[k.to(device="cuda", dtype=torch.bfloat16)],
                         v=[v.to(device="cuda", dtype=torch.bfloat16)])
        got = ops().paged_attention(q.to(device="cuda", dtype=torch.bfloat16), case.cache,
                                    case.meta([0], [(0, n)]), 1.0)
        for h in range(hq):
            want = case.v[0][far, h // 2].float().expand(n - far, d)
            torch.testing.assert_close(got[far:, h].float(), want, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_paged_attention_cut_and_batch_invariance(dtype):
    """The same query position gives close results (float32: the same bits)
    whatever the cut of the prompt and whatever else is in the batch
    (tests/test_03_extend_attention.py:75-152 of the reference)."""
    hq, hkv, d, page = 6, 2, 32, 16
    lens = [150, 97, 40]
    case = PagedCase(lens, hkv, d, page, dtype, seed=17)
    g = torch.Generator().manual_seed(18)
    qfull = torch.randn(150, hq, d, generator=g).to(device="cuda", dtype=dtype)
    whole = ops().paged_attention(qfull, case.cache, case.meta([0], [(0, 150)]), d ** -0.5)
    # cut at 70, and as one of three sequences
    other = torch.randn(97 - 10 + 40, hq, d, generator=g).to(device="cuda", dtype=dtype)
    part = ops().paged_attention(qfull[70:], case.cache, case.meta([0], [(70, 80)]), d ** -0.5)
    mixed_q = torch.cat([other[:87], qfull[70:], other[87:]])
    mixed = ops().paged_attention(mixed_q, case.cache,
                                  case.meta([1, 0, 2], [(10, 87), (70, 80), (0, 40)]), d ** -0.5)
    one = ops().paged_attention(qfull[149:150], case.cache, case.meta([0], [(149, 1)]), d ** -0.5)
    if dtype == torch.float32:
        assert torch.equal(part, whole[70:])
        assert torch.equal(mixed[87:167], whole[70:])
        assert torch.equal(one[0], whole[149])
    else:
        torch.testing.assert_close(part.float(), whole[70:].float(), **tol(dtype))
        torch.testing.assert_close(mixed[87:167].float(), whole[70:].float(), **tol(dtype))
        torch.testing.assert_close(one[0].float(), whole[149].float(), **tol(dtype))
    # running it again gives the same bits in either dtype
    again = ops().paged_attention(qfull, case.cache, case.meta([0], [(0, 150)]), d ** -0.5)
    assert torch.equal(again, whole)


# ------------------------------------------------------------------ sampling

def test_argmax_lowest_index_on_ties():
    logits = torch.zeros(3, 151936, device="cuda")
    logits[0, 7] = 5.0
    logits[1, 3] = 2.0
    logits[1, 151935] = 2.0
    logits[2, 151935] = 1.0
    assert ops().argmax(logits).tolist() == [7, 3, 151935]
    x = torch.randn(9, 1000, device="cuda")
    assert ops().argmax(x).tolist() == torch.argmax(x, -1).tolist()


@pytest.mark.parametrize("v,masked", [(5003, False), (151936, False), (20001, True), (8193, False)])
def test_gumbel_sample_matches_formula(v, masked):
    """Narrow rows take one block per row, wide rows a block per chunk of 4,096 ids
    (normaliser put together from the chunks, then the scores)."""
    torch.manual_seed(20)
    r = 16
    logits = 3 * torch.randn(r, v, device="cuda")
    temps = torch.tensor([0.0, 0.8, 1.5, 0.3] * 4, device="cuda")
    seeds = torch.arange(r, device="cuda", dtype=torch.int64) * 977 - 5
    pos = torch.arange(100, 100 + r, device="cuda", dtype=torch.int64)
    keep = (torch.rand(r, v, device="cuda") < 0.3).to(torch.uint8) if masked else None
    got = ops().gumbel_sample(logits, temps, seeds, pos, keep)
    scores = ref.gumbel_scores(logits, temps, seeds, pos, keep)
    want = ref.gumbel_sample(logits, temps, seeds, pos, keep)
    if masked:
        assert all(keep[i, got[i]] == 1 for i in range(r) if temps[i] > 0)
    for i in range(r):
        if got[i] != want[i]:      # only a near tie of the two scores may differ
            assert abs(float(scores[i, got[i]] - scores[i, want[i]])) < 1e-4, (i, got[i], want[i])
    assert (got == want).float().mean() > 0.9


@pytest.mark.parametrize("v", [5000, 151936])
def test_gumbel_draw_independent_of_batch_and_depends_on_position(v):
    torch.manual_seed(21)
    row = torch.randn(1, v, device="cuda")
    one = lambda lg, seeds, pos: ops().gumbel_sample(
        lg, torch.full((lg.shape[0],), 0.8, device="cuda"),
        torch.tensor(seeds, dtype=torch.int64, device="cuda"),
        torch.tensor(pos, dtype=torch.int64, device="cuda"))
    alone = one(row, [1234], [17])
    for batch in (2, 7, 33):
        lg = torch.cat([torch.randn(batch - 1, v, device="cuda"), row])
        toks = one(lg, [1234] * batch, list(range(100, 100 + batch - 1)) + [17])
        assert toks[-1] == alone[0]
    same = torch.randn(1, 1000, device="cuda").repeat(64, 1)
    assert len(set(one(same, [42] * 64, list(range(64))).tolist())) > 1


@pytest.mark.parametrize("v", [151936, 20001, 5000, 300])
def test_top_k_top_p_threshold_is_what_the_sort_rule_keeps(v):
    """The kernels keep {p >= threshold}; the threshold they find without a sort
    keeps what the reference's rule keeps (sort descending, drop when the mass before a
    token exceeds top_p or its rank reaches top_k), up to a token at the boundary whose
    probability the two computations round differently."""
    from tests.torch_kernels import keep_mask
    torch.manual_seed(23)
    r = 12
    logits = 4 * torch.randn(r, v, device="cuda")
    temps = torch.tensor([0.6, 0.6, 1.0, 0.8, 1.3, 0.0, 0.7, 0.6, 2.0, 0.6, 1.0, 0.9], device="cuda")
    top_ks = torch.tensor([20, -1, 50, 1, 7, 5, -1, 20, 1000, 3, -1, 40000], device="cuda", dtype=torch.int64)
    top_ps = torch.tensor([0.95, 0.9, 1.0, 0.5, 1.0, 0.9, 1.0, 1.0, 0.99, 0.2, 0.5, 0.999], device="cuda")
    seeds = torch.arange(r, device="cuda", dtype=torch.int64) + 11
    pos = torch.arange(50, 50 + r, device="cuda", dtype=torch.int64)
    toks, thr = ops().gumbel_sample(logits, temps, seeds, pos, top_ks=top_ks, top_ps=top_ps,
                                    return_thresholds=True)
    want_keep = keep_mask(logits, temps, top_ks, top_ps).bool()
    t_safe = torch.where(temps > 0, temps, torch.ones_like(temps))
    probs = torch.softmax(logits / t_safe.unsqueeze(-1), dim=-1)
    # The kept set is rebuilt here from torch's softmax, whose probabilities differ from the
    # kernels' own by a few units in the last place (another exponential, another order of
    # the normaliser's sum): the threshold, which IS the kernels' probability of the last
    # kept token, is compared with that much slack, or the rebuilt set would lose that token.
    mine = probs.view(torch.int32) >= (thr.unsqueeze(-1) - 16)
    for i in range(r):
        if temps[i] <= 0:
            assert toks[i] == logits[i].argmax() and thr[i] == 0
            continue
        if top_ks[i] <= 0 and top_ps[i] >= 1:
            assert thr[i] == 0
            continue
        differ = int((mine[i] ^ want_keep[i]).sum())
        assert differ <= 2, (i, differ, int(mine[i].sum()), int(want_keep[i].sum()))
        assert bool(mine[i, toks[i]]) or bool(want_keep[i, toks[i]])
    # the draw itself: the same as with the reference's mask wherever the two sets agree
    with_mask = ops().gumbel_sample(logits, temps, seeds, pos, want_keep.to(torch.uint8).contiguous())
    agree = [(mine[i] ^ want_keep[i]).sum() == 0 for i in range(r)]
    assert all(toks[i] == with_mask[i] for i in range(r) if agree[i]) and sum(map(bool, agree)) >= r - 3


def test_top_k_top_p_respected():
    from deterministic_inference_b200.config import SamplingParams
    from deterministic_inference_b200.sampling import sample
    logits = torch.tensor([[10.0, 9.0, 8.0, -20.0, -20.0]], device="cuda")
    for pos in range(100):
        tok = sample(logits, [SamplingParams(temperature=2.0, seed=5, top_k=3)], [pos]).item()
        assert tok in (0, 1, 2)
    peaked = torch.tensor([[10.0, 0.0, 0.0, 0.0, 0.0]], device="cuda")
    for pos in range(50):
        assert sample(peaked, [SamplingParams(temperature=1.0, seed=5, top_p=0.5)], [pos]).item() == 0


def test_no_cpu_path():
    from deterministic_inference_b200.kernels.ops import KernelError
    with pytest.raises(KernelError, match="CUDA"):
        ops().rms_norm(torch.randn(2, 8), torch.ones(8), 1e-6)


def test_sizes_outside_a_kernels_range_are_refused_with_a_clear_error():
    """What a kernel cannot take it refuses by name and size; it never runs on it."""
    from deterministic_inference_b200.kernels.ops import KernelError
    o = ops()
    dev = "cuda"
    # attention: heads of more than 256 elements
    d = 272
    q = torch.zeros(1, 2, d, device=dev)
    cache = torch.zeros(3, 2, 2, 16, d, device=dev)
    case_meta = PagedCase([4], 2, 16, 16, torch.float32, seed=1).meta([0], [(3, 1)])
    with pytest.raises(KernelError, match="head_dim 272"):
        o.paged_attention(q, cache, case_meta, 1.0)
    # query heads that the kv heads do not divide
    with pytest.raises(KernelError, match="q .* vs cache"):
        o.paged_attention(torch.zeros(1, 3, 16, device=dev), torch.zeros(3, 2, 2, 16, 16, device=dev),
                          case_meta, 1.0)
    # norm: a row wider than the widest kernel's shared memory, and a weight of another width
    with pytest.raises(KernelError, match="row width 70001"):
        o.rms_norm(torch.zeros(2, 70001, device=dev), torch.ones(70001, device=dev), 1e-6)
    with pytest.raises(KernelError, match="weight has 7 elements"):
        o.rms_norm(torch.zeros(2, 8, device=dev), torch.ones(7, device=dev), 1e-6)
    # rotation over an odd number of dimensions
    with pytest.raises(KernelError):
        o.qk_norm_rope_cache(torch.zeros(1, 4 * 16, device=dev), 2, 1, 16, None, None, 1e-6,
                             torch.zeros(8, 7, device=dev), torch.zeros(1, dtype=torch.int32, device=dev),
                             None, None, 16)
    # dtypes the package does not compute in
    with pytest.raises(KernelError, match="float32 or bfloat16|must be"):
        o.rms_norm(torch.zeros(2, 8, device=dev, dtype=torch.float16), torch.ones(8, device=dev), 1e-6)
    # a non-contiguous input is named, not silently copied
    with pytest.raises(KernelError, match="contiguous"):
        o.rms_norm(torch.zeros(8, 4, device=dev).t(), torch.ones(8, device=dev), 1e-6)


def test_a_wait_that_runs_out_ends_the_kernel_and_is_reported_once():
    """Every mbarrier wait of the package's kernels is bounded.  A test-only kernel waits
    one millisecond on a barrier that nothing arrives on (and that no copy targets): the
    launch ends by itself, its error word is set, ``ops.check_kernel_status`` raises a
    ``KernelError`` that names the library, clears the word, and the next check passes; a
    wait whose barrier is arrived on sets nothing."""
    import time
    from ctypes import c_int, c_ulonglong, c_void_p
    from pathlib import Path
    from deterministic_inference_b200.kernels import build
    from deterministic_inference_b200.kernels.ops import KernelError
    build.register_source("test_wait", Path(__file__).parent / "kernels" / "wait_runs_out.cu")
    lib = build.load_library("test_wait")
    ops().register_kernel_status("test_wait", lib.test_wait_status, lib.test_wait_status_clear)
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    try:
        ops().check_kernel_status()
        assert lib.test_wait_launch(c_ulonglong(1_000_000), c_int(1), stream) == 0
        torch.cuda.synchronize()
        ops().check_kernel_status()                       # the barrier was arrived on: nothing set
        t0 = time.perf_counter()
        assert lib.test_wait_launch(c_ulonglong(1_000_000), c_int(0), stream) == 0
        torch.cuda.synchronize()
        assert time.perf_counter() - t0 < 1.0             # it gave up after about a millisecond
        assert ops().kernel_status()["test_wait"] == 7
        with pytest.raises(KernelError, match="test_wait"):
            ops().check_kernel_status()
        assert ops().kernel_status()["test_wait"] == 0    # reported once, then cleared
        ops().check_kernel_status()
        # the context is as usable as before
        x = torch.ones(8, 64, device="cuda", dtype=torch.bfloat16)
        w = torch.ones(64, device="cuda", dtype=torch.float32)
        torch.testing.assert_close(ops().rms_norm(x, w, 1e-6).float(), torch.ones(8, 64, device="cuda"),
                                   atol=1e-2, rtol=1e-2)
    finally:
        from deterministic_inference_b200.kernels import ops as _ops
        _ops._extra_status.pop("test_wait", None)


@pytest.mark.parametrize("m,i,h,splits", [(8, 3072, 1024, 0), (1, 3072, 1024, 0), (50, 3072, 1024, 0),
                                          (16, 1536, 512, 3), (128, 768, 256, 1), (5, 12288, 4096, 0),
                                          (2, 160, 96, 2), (3, 200, 72, 0)])
def test_product_that_gates_while_it_loads_gives_the_bits_of_the_two_kernels(switches, monkeypatch, m, i, h, splits):
    """The down projection of a gated feed-forward whose [gate | up] product lies in memory
    as split-k partials: the kernel that sums the partials, gates and multiplies in one go
    (its token operand made in shared memory) against the gate kernel followed by the plain
    product: the same bits, whether its own k is split or not."""
    o = ops()
    torch.manual_seed(31)
    x = torch.randn(m, h, device="cuda").to(torch.bfloat16)
    w_gu = (0.05 * torch.randn(2 * i, h, device="cuda")).to(torch.bfloat16)
    w_down = (0.05 * torch.randn(h, i, device="cuda")).to(torch.bfloat16)
    if splits:
        switches.gemm(splits=splits)
    switches.gated("0")
    monkeypatch.setattr(o, "GATE_IN_PRODUCT_ROWS", 128)
    monkeypatch.setattr(o, "GATE_IN_PRODUCT_WIDTH", 1 << 20)
    deferred = o.gated_linear(x, w_gu)
    if not isinstance(deferred, o.GatedSplit):
        pytest.skip("the gate_up product of this shape is not split")
    fused = o.linear(deferred, w_down)
    plain = o.linear(deferred.tensor(), w_down)
    assert type(fused) is type(plain)
    assert torch.equal(o.as_tensor(fused), o.as_tensor(plain))
    if isinstance(fused, o.SplitSum):
        assert torch.equal(fused.parts, plain.parts)
    g, u = (x.float() @ w_gu.float().T).to(torch.bfloat16).float().chunk(2, dim=1)
    want = (g * torch.sigmoid(g) * u).to(torch.bfloat16).float() @ w_down.float().T
    torch.testing.assert_close(o.as_tensor(fused).float(), want, atol=3e-2 * float(want.abs().max()), rtol=3e-2)
    from deterministic_inference_b200.kernels import gemm_bf16
    assert gemm_bf16.status() == 0


@pytest.mark.parametrize("hq,hkv,d,page,window,lens", [
    (16, 8, 128, 16, None, [1, 33, 257, 700, 128, 2049, 5, 129]),
    (8, 2, 128, 32, 300, [513, 2, 1290]),
    (6, 3, 64, 16, None, [40, 2100, 129, 127]),
    (16, 8, 128, 16, None, [5000, 300]),
    (5, 5, 48, 16, None, [70, 200, 3])])
def test_product_that_merges_attention_splits_while_it_loads_gives_the_bits_of_the_two_kernels(
        switches, hq, hkv, d, page, window, lens):
    """The output projection after a decode-only attention step: the decode kernel leaves its
    per-split partial results, and the product merges them into its token operand; against
    the merge kernel followed by the plain product: the same bits (a few splits, more than
    16, a window that cuts splits off the front)."""
    o = ops()
    case = PagedCase(lens, hkv, d, page, torch.bfloat16, seed=81)
    meta = case.meta(list(range(len(lens))), [(n - 1, 1) for n in lens])
    g = torch.Generator().manual_seed(82)
    q = torch.randn(len(lens), hq, d, generator=g).to(device="cuda", dtype=torch.bfloat16)
    w_o = (0.05 * torch.randn(1024 if d >= 64 else 80, hq * d, generator=g)).to(device="cuda", dtype=torch.bfloat16)
    merged = o.paged_attention(q, case.cache, meta, d ** -0.5, window)
    plain = o.linear(o.merge_heads(merged), w_o)
    switches.attention(defer_merge=True)
    deferred = o.paged_attention(q, case.cache, meta, d ** -0.5, window, defer=True)
    assert isinstance(deferred, o.SplitAttention)
    assert torch.equal(deferred.tensor().view_as(merged), merged)
    fused = o.linear(o.merge_heads(deferred), w_o)
    assert type(fused) is type(plain)
    assert torch.equal(o.as_tensor(fused), o.as_tensor(plain))
    from deterministic_inference_b200.kernels import gemm_bf16
    assert gemm_bf16.status() == 0
    # a step that also holds a prompt portion is not deferred
    meta2 = case.meta([0, 1], [(lens[0] - 1, 1), (0, lens[1])]) if lens[1] > 1 else None
    if meta2 is not None:
        q2 = torch.randn(1 + lens[1], hq, d, generator=g).to(device="cuda", dtype=torch.bfloat16)
        assert isinstance(o.paged_attention(q2, case.cache, meta2, d ** -0.5, window, defer=True), torch.Tensor)


@pytest.mark.parametrize("m,n,k", [(129, 1024, 1024), (2048, 4096, 1024), (300, 6144, 1024), (1000, 1000, 512),
                                   (257, 264, 72), (130, 8, 200), (4096, 1024, 3072), (77, 512, 64)])
def test_linear_bf16_many_rows_own_kernel(m, n, k):
    """The package's persistent tcgen05 product for many rows (all of k in one pass) against
    a float32 product: row counts, widths and depths that are no multiples of the tile,
    several tiles per CTA; a row's bits are the same in a product of other row counts, and
    with each of the three tile shapes (128 x 128, 128 x 256, 256 x 256 by a pair of CTAs)."""
    from deterministic_inference_b200.kernels import gemm_bf16
    torch.manual_seed(41)
    x = torch.randn(m, k, device="cuda").to(torch.bfloat16)
    w = (0.05 * torch.randn(n, k, device="cuda")).to(torch.bfloat16)
    want = x.float() @ w.float().T
    got = gemm_bf16.linear_large(x, w, torch.bfloat16)
    try:
        for shape in (0, 1, 2):
            gemm_bf16.force_large_shape(shape)
            assert torch.equal(gemm_bf16.linear_large(x, w, torch.bfloat16), got), shape
            if shape == 2:
                assert torch.equal(gemm_bf16.linear_large(x, w, torch.float32).to(torch.bfloat16), got)
    finally:
        gemm_bf16.force_large_shape(-1)
    assert got is not None and got.shape == (m, n) and got.dtype == torch.bfloat16
    torch.testing.assert_close(got.float(), want, atol=2e-2 * float(want.abs().max()), rtol=2e-2)
    got32 = gemm_bf16.linear_large(x, w, torch.float32)
    torch.testing.assert_close(got32, want, atol=1e-3 * float(want.abs().max()), rtol=1e-3)
    assert torch.equal(got32.to(torch.bfloat16), got)
    # the same rows in a product of fewer rows, and at another place in it
    part = gemm_bf16.linear_large(x[40:140].contiguous(), w, torch.bfloat16) if m >= 140 else None
    if part is not None:
        assert torch.equal(part, got[40:140])
    assert ops().kernel_status().get("gemm_bf16_large", 0) == 0


@pytest.mark.parametrize("m,i,k", [(2048, 3072, 1024), (129, 200, 72), (700, 1536, 512), (4100, 4096, 264)])
def test_gated_product_many_rows_gives_the_bits_of_product_and_gate(m, i, k):
    """The many-rows product with the gate in its epilogue against the same product followed
    by the gate kernel: the same bits."""
    from deterministic_inference_b200.kernels import gemm_bf16
    torch.manual_seed(43)
    x = torch.randn(m, k, device="cuda").to(torch.bfloat16)
    w = (0.05 * torch.randn(2 * i, k, device="cuda")).to(torch.bfloat16)
    fused = gemm_bf16.gated_linear_large(x, w)
    two = ops().silu_mul(gemm_bf16.linear_large(x, w, torch.bfloat16))
    assert fused is not None and torch.equal(fused, two)
    try:
        for shape in (0, 1, 2):   # one CTA on 128 tokens and 64 + 64 or 128 + 128 weight rows; a pair of CTAs on 256
            gemm_bf16.force_large_shape(shape)
            assert torch.equal(gemm_bf16.gated_linear_large(x, w), fused), shape
    finally:
        gemm_bf16.force_large_shape(-1)
    assert ops().kernel_status().get("gemm_bf16_large", 0) == 0
    y = (x.float() @ w.float().T).to(torch.bfloat16).float()
    want = y[:, :i] * torch.sigmoid(y[:, :i]) * y[:, i:]
    torch.testing.assert_close(fused.float(), want, atol=2e-2 * float(want.abs().max()), rtol=3e-2)


@pytest.mark.parametrize("t,hq,hkv,k,page_size,norm,rope", [
    (2048, 16, 8, 1024, 16, True, True), (300, 4, 2, 256, 16, True, True), (130, 8, 1, 384, 32, False, True),
    (700, 5, 5, 200, 8, True, False), (257, 3, 1, 72, 64, False, False)])
def test_qkv_projection_with_the_norms_in_its_epilogue_gives_the_bits_of_the_two_kernels(t, hq, hkv, k, page_size,
                                                                                         norm, rope):
    """The fused q/k/v projection of many bfloat16 rows whose epilogue norms q and k, rotates them
    and writes k and v to the cache (one kernel; tiles of one head and of two on one CTA, of two on a pair of CTAs),
    against the same product followed by the q/k kernel: the same q rows and the same cache,
    bit for bit; with and without norm weights and a rotation, an odd number of heads (the
    last tile's second half lies beyond them), token counts and depths off the tile's sizes,
    slots spread over pages, some tokens without a slot."""
    from deterministic_inference_b200.kernels import gemm_bf16
    o = ops()
    torch.manual_seed(53)
    d = 128
    x = torch.randn(t, k, device="cuda").to(torch.bfloat16)
    w = (0.08 * torch.randn((hq + 2 * hkv) * d, k, device="cuda")).to(torch.bfloat16)
    qn = (1 + 0.1 * torch.randn(d, device="cuda")) if norm else None
    kn = (1 + 0.1 * torch.randn(d, device="cuda")) if norm else None
    max_pos = 4096
    table = None
    if rope:
        inv = 1.0 / (10000.0 ** (torch.arange(0, d // 2, dtype=torch.float32, device="cuda") / (d // 2)))
        fr = torch.outer(torch.arange(max_pos, dtype=torch.float32, device="cuda"), inv)
        table = torch.cat([fr.cos(), fr.sin()], dim=-1).contiguous()
    positions = torch.randint(0, max_pos, (t,), device="cuda", dtype=torch.int32)
    pages = -(-t // page_size) + 3
    slots = torch.randperm((pages - 1) * page_size, device="cuda")[:t].to(torch.int32) + page_size
    slots[::17] = -1                                        # tokens whose keys are not cached
    want_cache = torch.full((pages, 2, hkv, page_size, d), 7.0, device="cuda", dtype=torch.bfloat16)
    want_q = o.qk_norm_rope_cache(gemm_bf16.linear_large(x, w, torch.bfloat16), hq, hkv, d, qn, kn, 1e-6, table,
                                  positions, want_cache, slots, page_size)
    try:
        for shape in (0, 1, 2):
            gemm_bf16.force_large_shape(shape)
            cache = torch.full_like(want_cache, 7.0)
            q = gemm_bf16.qkv_large(x, w, hq, hkv, qn, kn, 1e-6, table, positions, cache, slots, page_size)
            assert q is not None and torch.equal(q, want_q), shape
            assert torch.equal(cache, want_cache), shape
    finally:
        gemm_bf16.force_large_shape(-1)
    assert o.kernel_status().get("gemm_bf16_large", 0) == 0
    # against float32 arithmetic on the rounded product
    y = (x.float() @ w.float().T).to(torch.bfloat16).float().view(t, hq + 2 * hkv, d)
    qf = y[:, :hq]
    if norm:
        qf = qf * torch.rsqrt(qf.pow(2).mean(-1, keepdim=True) + 1e-6) * qn
    if rope:
        cs = table[positions.long()]
        c, s = cs[:, None, :d // 2], cs[:, None, d // 2:]
        a, b = qf[..., :d // 2], qf[..., d // 2:]
        qf = torch.cat([a * c - b * s, b * c + a * s], dim=-1)
    torch.testing.assert_close(want_q.float(), qf, atol=3e-2 * float(qf.abs().max()), rtol=3e-2)
