"""bfloat16 tensor-core attention over the paged cache: the split-KV decode
kernels for the batch's leading one-token sequences and the extend kernel for
sequences that bring a portion of a prompt.  ``supports`` says whether the
kernels take a shape; shapes they refuse run on the generic kernel.

The decode kernel writes per-split partial outputs to scratch memory
(``part_o`` float32 [sequences, heads, splits, head_dim] and ``part_lse``
[sequences, heads, splits]) which its second stage merges in split order.
"""

from __future__ import annotations

import os
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

SPLIT = 128        # keys per split of the decode kernel (fixed: the order of a
                   # sequence's reduction depends on its own length only)
TILE_ROWS = 64     # rows (token, head-of-group pairs) per tile of the mma.sync extend kernel
TC_TILE_ROWS = 128  # ... of the tcgen05 extend kernel (head_dim 128)


def supports(num_heads: int, num_kv_heads: int, head_dim: int, page_size: int) -> bool:
    group = num_heads // num_kv_heads
    return head_dim % 16 == 0 and 16 <= head_dim <= 128 and group <= 16 and num_kv_heads <= 65535


# A prompt's key range is cut at every multiple of CHUNK_TILES key tiles of 128 (chunks
# anchored at key 0, a constant size): a query tile whose keys reach beyond a cut is worked
# on by one CTA per chunk and a second kernel adds their partial results in chunk order.
# The cuts depend on positions alone, never on the step, so a token's bits do not either.
CHUNK_TILES = 32
MAX_CHUNKS = 16     # chunks the merge kernel adds for one row: 65,536 keys

# Switches for measurements and tests, read ONCE when the module is imported (the
# environment is not looked at again); tests set the entries of this dictionary.
#   decode_tma   0: keys copied row by row instead of page-wise by TMA
#   decode_pipe  0: one split per CTA; 1: one CTA per SM walks the splits, copies pipelined;
#                2: the latter when the step has more splits than CTAs that run at once
#   prefill_tc   0: mma.sync kernel; 1: one query tile per CTA; 2: two
#   prefill_pair auto | 0: every tile alone | 1: pairs from both ends | 2: neighbours
#   defer_merge  True: decode-only steps leave the merge of the splits to the output projection
SWITCHES = {
    "decode_tma": os.environ.get("DIB200_DECODE_TMA", "1") != "0",
    "decode_pipe": int(os.environ.get("DIB200_DECODE_PIPE", "2")),
    "prefill_tc": os.environ.get("DIB200_PREFILL_TC", "2"),
    "prefill_pair": os.environ.get("DIB200_PREFILL_PAIR", "auto"),
    # 1: a decode-only step's attention leaves its splits unmerged and the output projection
    # merges them while it loads its operand (the same bits; measured slower than the merge
    # kernel on B200, so off)
    "defer_merge": os.environ.get("DIB200_DEFER_MERGE", "0") == "1",
}

_sms: dict = {}


def _sm_count(device) -> int:
    n = _sms.get(device)
    if n is None:
        n = torch.cuda.get_device_properties(device).multi_processor_count
        _sms[device] = n
    return n


def extend_chunk_units(q_lens: list, kv_lens: list, first_seq: int, tokens_per_tile: int,
                       chunk_tiles: int):
    """(sequence, first token of A, of B, chunk) for every chunk of ``chunk_tiles`` key tiles
    that a pair of consecutive query tiles may need: chunks 0 .. the one of the pair's last
    position, with the lengths the host knows (under a captured graph an upper bound: a
    chunk past the real range costs a CTA that leaves at once).  Longest first, so that the
    CTAs the GPU takes up last are the short ones."""
    units = []
    span = chunk_tiles * 128
    for s in range(first_seq, len(q_lens)):
        prefix = kv_lens[s] - q_lens[s]
        for t0 in range(0, q_lens[s], 2 * tokens_per_tile):
            t1 = t0 + tokens_per_tile if t0 + tokens_per_tile < q_lens[s] else -1
            last_pos = prefix + min(t0 + 2 * tokens_per_tile, q_lens[s]) - 1
            for c in range(last_pos // span + 1):
                keys = min(last_pos + 1, (c + 1) * span) - c * span
                units.append((-keys, s, t0, t1, c))
    units.sort()
    # the kernel takes its list from the end (the last entry first)
    units.reverse()
    return [u[1] for u in units], [u[2] for u in units], [u[3] for u in units], [u[4] for u in units]


def extend_tile_pairs(q_lens: list, kv_lens: list, first_seq: int, tokens_per_tile: int,
                      window: int, alone: bool = False, neighbours: bool = False):
    """(sequence, first token of A, first token of B or -1) for the CTAs of the kernel
    that takes two query tiles of a sequence at once.  Under a causal mask the k-th tile
    of a prompt needs about k key tiles more than the first, so the k-th tile is paired
    with the k-th from the end: every pair then needs the same number of key-tile products,
    and the short tile's key tiles are among the long one's.  With a window every tile
    needs about as many key tiles as the next, and neighbours share most of them: they
    are paired.  ``neighbours``: neighbours are paired under a causal mask too, for steps
    with more CTAs than SMs: the GPU then evens the CTAs out by itself (the longest come
    first), and neighbours read each key tile once for both, where a pair from both ends
    reads the long tile's keys for one tile most of the time (one layer of 16 + 8 heads:
    3,072 tokens 66 us against 81 us, 8,192 tokens 290 us against 347 us; but 2,048 tokens,
    one CTA per SM at most, 47 us against 36 us).  ``alone``: every tile gets a CTA of its own (B = -1), for steps with so few
    tiles that pairs would leave most of the GPU idle; the kernel then keeps two key tiles
    of that one query tile in flight.  The entries are sorted by the key tiles they need,
    the longest last (the kernel takes its list from the end)."""
    units = []
    for s in range(first_seq, len(q_lens)):
        prefix = kv_lens[s] - q_lens[s]
        starts = list(range(0, q_lens[s], tokens_per_tile))
        n = len(starts)
        if alone:
            pairs = [(a, -1) for a in starts]
        elif window > 0 or neighbours:
            pairs = [(starts[i], starts[i + 1] if i + 1 < n else -1) for i in range(0, n, 2)]
        else:
            pairs = [(starts[i], starts[n - 1 - i] if n - 1 - i > i else -1) for i in range((n + 1) // 2)]
        for a, b in pairs:
            last = prefix + min(max(a, b) + tokens_per_tile, q_lens[s]) - 1
            first = max(0, prefix + a - window + 1) if window > 0 else 0
            units.append((last // 128 - first // 128 + 1, s, a, b))
    units.sort()
    return [u[1] for u in units], [u[2] for u in units], [u[3] for u in units]


def extend_tiles(q_lens: list, first_seq: int, tokens_per_tile: int):
    seqs, starts = [], []
    for s in range(first_seq, len(q_lens)):
        for t0 in range(0, q_lens[s], tokens_per_tile):
            seqs.append(s)
            starts.append(t0)
    return seqs, starts


def _pair_lists(meta, nd: int, tpt: int, window: int, hkv: int, max_chunks: int, t: int, hq: int,
                d: int, device):
    """The CTA list of the two-tile prompt kernel for this step, on the device: (sequences,
    first tokens of A, count, first tokens of B), the chunk of each entry (or None) and
    the scratch for partial results (or Nones).  How tiles are paired depends on the step
    (few tiles: each alone; more CTAs than SMs: neighbours; else from both ends); the
    arithmetic of a tile does not depend on its partner."""
    if max_chunks > 1:
        seqs, starts, starts_b, chunks = extend_chunk_units(meta.q_lens, meta.kv_lens, nd, tpt,
                                                            CHUNK_TILES)
        both = torch.tensor([seqs, starts, chunks, starts_b], dtype=torch.int32).to(device, non_blocking=True)
        ws = (torch.empty(t, hq, max_chunks, d, dtype=torch.float32, device=device),
              torch.empty(t, hq, max_chunks, 2, dtype=torch.float32, device=device))
        return (both[0], both[1], len(seqs), both[3]), both[2], ws
    n_tiles = sum(-(-n // tpt) for n in meta.q_lens[nd:])
    ctas = (n_tiles + 1) // 2 * hkv
    how = SWITCHES["prefill_pair"]
    alone = how == "0" or (how == "auto" and ctas * 2 <= _sm_count(device))
    neighbours = how == "2" or (how == "auto" and ctas > _sm_count(device))
    seqs, starts, starts_b = extend_tile_pairs(meta.q_lens, meta.kv_lens, nd, tpt, window, alone, neighbours)
    both = torch.tensor([seqs, starts, starts_b], dtype=torch.int32).to(device, non_blocking=True)
    return (both[0], both[1], len(seqs), both[2]), None, (None, None)


def run(q, out, kv_cache, meta, scale: float, window: int, defer: bool = False):
    """Fills ``out``; or, with ``defer`` and a step of one-token sequences only, returns an
    ``ops.SplitAttention`` (the decode kernel's partial results, not merged) and leaves
    ``out`` alone."""
    from .ops import SplitAttention, _check, _lib, _ptr, _stream

    lib = _lib("attention_bf16")
    t, hq, d = q.shape
    _, _, hkv, page_size, _ = kv_cache.shape
    nd, b = meta.num_decode, len(meta.q_lens)
    bt = meta.block_table
    if nd > 0:
        max_splits = max(1, -(-max(meta.kv_lens[:nd]) // SPLIT))
        ws = meta.scratch.get(("decode_ws", hq, d, max_splits))
        if ws is None:
            ws = (torch.empty(nd, hq, max_splits, d, dtype=torch.float32, device=q.device),
                  torch.empty(nd, hq, max_splits, dtype=torch.float32, device=q.device))
            meta.scratch[("decode_ws", hq, d, max_splits)] = ws
        use_tma, pipelined = SWITCHES["decode_tma"], SWITCHES["decode_pipe"]
        deferred = defer and nd == b and SWITCHES["defer_merge"]
        st = lib.dib_decode_attention_bf16(
            _ptr(q), c_void_p(0) if deferred else _ptr(out), _ptr(kv_cache),
            c_longlong(kv_cache.shape[0] if use_tma else 0),
            _ptr(bt), c_int(bt.shape[1]), _ptr(meta.seq_lens),
            _ptr(ws[0]), _ptr(ws[1]), c_int(nd), c_int(max_splits), c_int(hq), c_int(hkv), c_int(d),
            c_int(page_size), c_float(scale), c_int(window), c_int(pipelined), _stream())
        _check(st, "decode_attention_bf16", f"heads {hq}/{hkv}, head_dim {d}", kernels=1 if deferred else 2)
        if deferred:
            return SplitAttention(ws[0], ws[1], meta.seq_lens, nd, window, q.dtype)
    group = hq // hkv
    tc_mode = SWITCHES["prefill_tc"]
    if b > nd and d == 128 and TC_TILE_ROWS % group == 0 and page_size in (8, 16, 32, 64, 128) \
            and tc_mode != "0":
        # tcgen05 kernels: 128 rows per query tile, one or two tiles per CTA
        pair = tc_mode != "1"
        tpt = TC_TILE_ROWS // group
        tc_lib = _lib("attention_prefill_tc")
        if not pair:
            tiles = meta.scratch.get(("extend_tiles", tpt))
            if tiles is None:
                seqs, starts = extend_tiles(meta.q_lens, nd, tpt)
                both = torch.tensor([seqs, starts], dtype=torch.int32).to(q.device, non_blocking=True)
                tiles = (both[0], both[1], len(seqs))
                meta.scratch[("extend_tiles", tpt)] = tiles
            st = tc_lib.dib_extend_attention_tc(
                _ptr(q), _ptr(out), _ptr(kv_cache), c_longlong(kv_cache.shape[0]), _ptr(bt),
                c_int(bt.shape[1]), _ptr(meta.cu_q_lens), _ptr(meta.seq_lens), _ptr(tiles[0]),
                _ptr(tiles[1]), c_int(tiles[2]), c_int(hq), c_int(hkv), c_int(d), c_int(page_size),
                c_float(scale), c_int(window), _stream())
            _check(st, "extend_attention_tc", f"heads {hq}/{hkv}, head_dim {d}")
            return
        # The lengths the host knows (under a captured graph an upper bound) say how many
        # chunks the launch must provide for; which chunks a row's result is added from
        # follows from its position alone (see CHUNK_TILES).
        n_keys = max(meta.kv_lens[nd:])
        max_chunks = -(-n_keys // (CHUNK_TILES * 128))
        if max_chunks <= MAX_CHUNKS:
            got = meta.scratch.get(("extend_pairs", tpt, window > 0))
            if got is None:
                got = _pair_lists(meta, nd, tpt, window, hkv, max_chunks, t, hq, d, q.device)
                meta.scratch[("extend_pairs", tpt, window > 0)] = got
            tiles, chunk_list, ws = got
            st = tc_lib.dib_extend_attention_tc_pair(
                _ptr(q), _ptr(out), _ptr(kv_cache), c_longlong(kv_cache.shape[0]), _ptr(bt),
                c_int(bt.shape[1]), _ptr(meta.cu_q_lens), _ptr(meta.seq_lens), _ptr(tiles[0]),
                _ptr(tiles[1]), _ptr(tiles[3]), c_int(tiles[2]), c_int(hq), c_int(hkv), c_int(d),
                c_int(page_size), c_float(scale), c_int(window), c_int(CHUNK_TILES if max_chunks > 1 else 0),
                _ptr(chunk_list), c_int(max_chunks), _ptr(ws[0]), _ptr(ws[1]), _ptr(meta.token_seq),
                c_int(nd), c_int(t - nd), _stream())
            _check(st, "extend_attention_tc_pair", f"heads {hq}/{hkv}, head_dim {d}",
                   kernels=2 if max_chunks > 1 else 1)
            return
        # longer than the merge kernel takes: the mma.sync kernel below
    if b > nd:
        tpt = TILE_ROWS // (hq // hkv)
        tiles = meta.scratch.get(("extend_tiles", tpt))
        if tiles is None:
            seqs, starts = extend_tiles(meta.q_lens, nd, tpt)
            both = torch.tensor([seqs, starts], dtype=torch.int32).to(q.device, non_blocking=True)
            tiles = (both[0], both[1], len(seqs))
            meta.scratch[("extend_tiles", tpt)] = tiles
        st = lib.dib_extend_attention_bf16(
            _ptr(q), _ptr(out), _ptr(kv_cache), _ptr(bt), c_int(bt.shape[1]), _ptr(meta.cu_q_lens),
            _ptr(meta.seq_lens), _ptr(tiles[0]), _ptr(tiles[1]), c_int(tiles[2]), c_int(hq),
            c_int(hkv), c_int(d), c_int(page_size), c_float(scale), c_int(window), _stream())
        _check(st, "extend_attention_bf16", f"heads {hq}/{hkv}, head_dim {d}")
