"""The batch of one step: a flat list of tokens from several sequences.

The reference builds one ``ForwardBatch`` per mode (prefill of whole prompts, or
one decode token per request) with CSR index lists of every cached token
(sid/engine/batch.py:30-154).  Here one batch holds any mix: each sequence
contributes ``q_len >= 1`` new tokens at positions ``num_computed ..
num_computed + q_len - 1``, portions of prompts beside single decoded tokens;
the cache is addressed through block tables, not per-token lists.  Sequences
with one token come first, so the decode kernel and the prefill kernel each take
a contiguous range.

All integer metadata of a step is packed into one host array and reaches the
device in one copy.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import numpy as np
import torch


@dataclass
class SequenceInput:
    """One sequence's share of a step."""

    slot: int                 # the request's state slot
    tokens: list              # its next tokens
    num_computed: int         # tokens of it already in the cache
    want: list = field(default_factory=list)   # places among ``tokens`` whose logits are wanted
    pending_row: int = -1     # >= 0: the LAST of ``tokens`` is not known on the host; it is row
                              # ``pending_row`` of the tokens the previous step sampled


@dataclass
class AttentionMeta:
    """Per cache group: where this step's keys go and where a sequence's keys lie;
    plus the batch-wide sequence description every attention kernel needs."""

    block_table: torch.Tensor        # int32 [B, max_blocks]
    slot_mapping: torch.Tensor       # int32 [T]
    token_seq: torch.Tensor          # int32 [T] sequence index of each token
    positions: torch.Tensor          # int32 [T]
    cu_q_lens: torch.Tensor          # int32 [B+1]
    seq_lens: torch.Tensor           # int32 [B]  keys per sequence after this step
    q_lens: list                     # host copies
    kv_lens: list
    num_decode: int                  # leading sequences with exactly one token
    scratch: dict = field(default_factory=dict)   # per-step data kernels derive (tile lists)


@dataclass
class StepBatch:
    num_tokens: int
    num_seqs: int
    num_decode: int
    num_logits: int
    input_ids: torch.Tensor          # int32 [T]
    positions: torch.Tensor          # int32 [T]
    token_seq: torch.Tensor          # int32 [T]
    cu_q_lens: torch.Tensor          # int32 [B+1]
    seq_lens: torch.Tensor           # int32 [B]
    state_slots: torch.Tensor        # int32 [B]
    logit_indices: torch.Tensor      # int32 [R] rows of the token list
    q_lens: list
    kv_lens: list
    slots: list                      # host copy of state_slots
    groups: dict                     # group key -> AttentionMeta
    logit_rows: list                 # per input entry (caller's order): its rows of the logits
    order: list                      # batch order -> index of the caller's entry
    patch_dst: Optional[torch.Tensor] = None   # int32 [B]: place in input_ids, or -1
    patch_src: Optional[torch.Tensor] = None   # int32 [B]: row of the previous step's tokens
    num_patches: int = 0
    logits_of_all_rows: bool = False            # every token's logits are wanted, in the tokens' order


def _align(n: int, a: int = 4) -> int:
    return (n + a - 1) // a * a


class PackedLayout:
    """Where each piece of a step's integer metadata lies in the one packed int32
    array, for ``t`` tokens, ``b`` sequences, ``r`` logit rows and block tables
    ``width`` pages wide in each of ``num_groups`` cache groups."""

    def __init__(self, t: int, b: int, r: int, width: int, num_groups: int):
        self.t, self.b, self.r, self.width, self.num_groups = t, b, r, width, num_groups
        self.off = {}
        cur = 0
        for name, n in (("input_ids", t), ("positions", t), ("token_seq", t), ("cu_q_lens", b + 1),
                        ("seq_lens", b), ("state_slots", b), ("logit_indices", r),
                        ("patch_dst", b), ("patch_src", b)):
            self.off[name] = (cur, n)
            cur = _align(cur + n)
        for gi in range(num_groups):
            self.off[("bt", gi)] = (cur, b * width)
            cur = _align(cur + b * width)
            self.off[("sm", gi)] = (cur, t)
            cur = _align(cur + t)
        self.size = max(cur, 1)

    def seg(self, array, name):
        s, n = self.off[name]
        return array[s:s + n]


def step_views(td: torch.Tensor, lay: PackedLayout, group_list: list, q_lens: list, kv_lens: list,
               slots: list, num_decode: int, logit_rows: list, order: list) -> "StepBatch":
    """A ``StepBatch`` whose tensors are views of the packed device array ``td``."""
    b = lay.b
    groups = {}
    for gi, g in enumerate(group_list):
        groups[g.key] = AttentionMeta(
            block_table=lay.seg(td, ("bt", gi)).view(b, lay.width),
            slot_mapping=lay.seg(td, ("sm", gi)), token_seq=lay.seg(td, "token_seq"),
            positions=lay.seg(td, "positions"), cu_q_lens=lay.seg(td, "cu_q_lens"),
            seq_lens=lay.seg(td, "seq_lens"), q_lens=q_lens, kv_lens=kv_lens, num_decode=num_decode)
    return StepBatch(
        num_tokens=lay.t, num_seqs=b, num_decode=num_decode, num_logits=lay.r,
        input_ids=lay.seg(td, "input_ids"), positions=lay.seg(td, "positions"),
        token_seq=lay.seg(td, "token_seq"), cu_q_lens=lay.seg(td, "cu_q_lens"),
        seq_lens=lay.seg(td, "seq_lens"), state_slots=lay.seg(td, "state_slots"),
        logit_indices=lay.seg(td, "logit_indices"), q_lens=q_lens, kv_lens=kv_lens, slots=slots,
        groups=groups, logit_rows=logit_rows, order=order,
        patch_dst=lay.seg(td, "patch_dst"), patch_src=lay.seg(td, "patch_src"),
        # one-token sequences that all want their logits: row i of the logits is token i
        logits_of_all_rows=(num_decode == b and lay.t == b and lay.r == b))


@dataclass
class StepShape:
    """What a step's entries come to, before anything is packed: the batch order (one-token
    sequences first), lengths, where the wanted logits lie."""
    order: list            # batch order -> index of the caller's entry
    seqs: list             # the entries in batch order
    q_lens: list
    kv_lens: list
    num_decode: int
    t: int                 # tokens of the step
    logit_rows: list       # per caller's entry: its rows of the logits
    logit_index: list      # per logits row: its row of the token list
    slots: list
    width: int             # pages of the longest sequence


def describe_step(entries: list, cache) -> StepShape:
    if not entries:
        raise ValueError("a step needs at least one sequence")
    for e in entries:
        if len(e.tokens) < 1:
            raise ValueError("every sequence of a step brings at least one token")
        for w in e.want:
            if not 0 <= w < len(e.tokens):
                raise ValueError(f"wanted place {w} is outside the {len(e.tokens)} tokens given")
    order = sorted(range(len(entries)), key=lambda i: (len(entries[i].tokens) != 1, i))
    seqs = [entries[i] for i in order]
    q_lens = [len(e.tokens) for e in seqs]
    kv_lens = [e.num_computed + len(e.tokens) for e in seqs]
    logit_rows: list = [None] * len(entries)
    logit_index: list = []
    start = 0
    for bi, e in enumerate(seqs):
        rows = []
        for w in e.want:
            rows.append(len(logit_index))
            logit_index.append(start + w)
        logit_rows[order[bi]] = rows
        start += q_lens[bi]
    return StepShape(order=order, seqs=seqs, q_lens=q_lens, kv_lens=kv_lens,
                     num_decode=sum(1 for q in q_lens if q == 1), t=sum(q_lens),
                     logit_rows=logit_rows, logit_index=logit_index, slots=[e.slot for e in seqs],
                     width=max(1, max(-(-kv // cache.page_size) for kv in kv_lens)))


def fill_packed(host: np.ndarray, lay: PackedLayout, shape: StepShape, cache, group_list: list) -> int:
    """Write the step's integer metadata into the packed array ``host`` laid out by
    ``lay`` (block tables ``lay.width`` >= ``shape.width`` pages wide).  Returns the number
    of tokens that are to be patched in from the previous step's samples.

    ``lay`` may hold more sequences and more tokens than the step has (a captured graph is
    made for a bucket of sizes): the rest are padding sequences that live on page 0 and
    state slot 0, which no request owns.  Each of them brings one token, except the last,
    which brings what is left of the layout's tokens (none, perhaps); their tokens have id 0,
    positions inside page 0 and a key count of their own token count (1 at least).  The
    padding rows follow the step's own rows, so no row of a request moves.  If the layout
    has more logits rows than the step wants, each padding sequence asks for one, which the
    caller drops.  An entry of the step itself may be a padding sequence too (state slot 0,
    which no request has: the step graphs add one-token entries of that kind to fill a bucket
    of decode sequences); it gets an all-zero block table and cache slot 0 like the others."""
    host[:] = 0
    seqs, q_lens = shape.seqs, shape.q_lens
    n_pad = lay.b - len(seqs)
    pad_t = lay.t - shape.t
    if n_pad < 0 or pad_t < 0 or (n_pad == 0 and pad_t != 0) or pad_t < n_pad - 1 \
            or lay.r - len(shape.logit_index) not in (0, n_pad):
        raise ValueError(f"layout of {lay.b} sequences / {lay.t} tokens does not fit a step of "
                         f"{len(seqs)} sequences / {shape.t} tokens")
    ids, pos, tseq = lay.seg(host, "input_ids"), lay.seg(host, "positions"), lay.seg(host, "token_seq")
    cu = lay.seg(host, "cu_q_lens")
    pdst, psrc = lay.seg(host, "patch_dst"), lay.seg(host, "patch_src")
    pdst[:] = -1
    num_patches = 0
    start = 0
    for bi, e in enumerate(seqs):
        q = q_lens[bi]
        if q == 1:
            ids[start] = e.tokens[0]
            pos[start] = e.num_computed
        else:
            ids[start:start + q] = e.tokens
            pos[start:start + q] = np.arange(e.num_computed, e.num_computed + q)
        tseq[start:start + q] = bi
        start += q
        cu[bi + 1] = start
        if e.pending_row >= 0:
            pdst[bi] = start - 1                 # the sequence's last token
            psrc[bi] = e.pending_row
            num_patches += 1
    n = len(seqs)
    lay.seg(host, "seq_lens")[:n] = shape.kv_lens
    lay.seg(host, "state_slots")[:n] = shape.slots
    lay.seg(host, "logit_indices")[:len(shape.logit_index)] = shape.logit_index
    if n_pad:
        counts = np.ones(n_pad, dtype=np.int64)
        counts[-1] = pad_t - (n_pad - 1)
        ends = start + np.cumsum(counts)
        tseq[start:] = np.repeat(np.arange(n, lay.b), counts)
        last = int(counts[-1])
        if last > 1:      # the last one's tokens: positions that stay inside page 0
            pos[lay.t - last:] = np.arange(last) % min(g.page_size for g in group_list)
        cu[n + 1:] = ends
        lay.seg(host, "seq_lens")[n:] = np.maximum(counts, 1)
        if lay.r > len(shape.logit_index):
            lay.seg(host, "logit_indices")[len(shape.logit_index):] = np.minimum(ends - counts, lay.t - 1)
    for gi, g in enumerate(group_list):
        bt = lay.seg(host, ("bt", gi)).reshape(lay.b, lay.width)
        sm = lay.seg(host, ("sm", gi))
        ps = g.page_size
        start = 0
        for bi, e in enumerate(seqs):
            if e.slot == 0:          # a padding sequence given as an entry: page 0, cache slot 0
                start += q_lens[bi]
                continue
            pl = g.pages[e.slot]
            m = min(len(pl), lay.width)
            bt[bi, :m] = pl[:m]
            q = q_lens[bi]
            if q == 1:
                page = pl[e.num_computed // ps]
                if page == 0:
                    raise ValueError(f"slot {e.slot}: position {e.num_computed} is not covered by a page")
                sm[start] = page * ps + e.num_computed % ps
            else:
                sm[start:start + q] = cache.slot_mapping(g, e.slot, e.num_computed, q)
            start += q
    return num_patches


class StepCheckError(ValueError):
    """A step's metadata names something outside its range (debug checks)."""


def check_packed(host: np.ndarray, lay: PackedLayout, cache, group_list: list, vocab_size: int,
                 max_positions: int, num_prev_tokens: int = 0) -> None:
    """Debug check of a step's packed metadata, on the host, before it reaches the device:
    every index a kernel will follow (token ids, positions, block-table entries, cache
    slots, logit rows, state slots, patch places) lies inside what it indexes.  The kernels
    read nothing else that a request controls, so this covers their read side; the
    reference checks its launch arguments on the host in the same spirit
    (sid/csrc/flash_decode.cu:298-345).  Raises ``StepCheckError`` naming the first
    offender."""
    def need(ok, what):
        if not ok:
            raise StepCheckError(f"step metadata: {what}")

    t, b = lay.t, lay.b
    ids, pos = lay.seg(host, "input_ids"), lay.seg(host, "positions")
    need(t == 0 or (ids.min() >= 0 and ids.max() < vocab_size),
         f"a token id outside [0, {vocab_size})")
    need(t == 0 or (pos.min() >= 0 and pos.max() < max_positions),
         f"a position outside [0, {max_positions})")
    tseq = lay.seg(host, "token_seq")
    need(t == 0 or (tseq.min() >= 0 and tseq.max() < b), "a token names a sequence the step does not have")
    cu = lay.seg(host, "cu_q_lens")
    slots = lay.seg(host, "state_slots")
    need(cu[0] == 0 and cu[b] == t and bool((np.diff(cu) >= np.where(slots == 0, 0, 1)).all()),
         "sequence boundaries do not cover the tokens, or a request's sequence brings none")
    lens = lay.seg(host, "seq_lens")
    need(bool((lens >= np.diff(cu)).all()) and (b == 0 or lens.max() <= cache.max_seq_len),
         "a sequence's key count is below its new tokens or beyond max_seq_len")
    need(b == 0 or (slots.min() >= 0 and slots.max() < cache.max_reqs), "a state slot outside the table")
    li = lay.seg(host, "logit_indices")
    need(li.size == 0 or (li.min() >= 0 and li.max() < t), "a logits row names a token the step does not have")
    pdst, psrc = lay.seg(host, "patch_dst"), lay.seg(host, "patch_src")
    live = pdst >= 0
    need(bool((pdst[live] < t).all()) and bool((psrc[live] >= 0).all())
         and bool((psrc[live] < max(num_prev_tokens, 1)).all()),
         "a token to be taken from the previous step's samples is out of range")
    for gi, g in enumerate(group_list):
        bt = lay.seg(host, ("bt", gi)).reshape(b, lay.width)
        need(bt.size == 0 or (bt.min() >= 0 and bt.max() < g.num_pages),
             f"group {g.key}: a block-table entry outside the pool of {g.num_pages} pages")
        sm = lay.seg(host, ("sm", gi))
        need(sm.size == 0 or (sm.min() >= 0 and sm.max() < g.num_pages * g.page_size),
             f"group {g.key}: a cache slot outside the pool")
        # pages a sequence needs for its keys must be real ones, except those a window gave back
        for bi in range(b):
            if slots[bi] == 0:
                continue        # a padding sequence: it lives on page 0 and slot 0 on purpose
            first_needed = 0
            if g.window is not None:
                first_needed = max(0, int(lens[bi]) - int(cu[bi + 1] - cu[bi]) - g.window + 1) // g.page_size
            need_pages = -(-int(lens[bi]) // g.page_size)
            row = bt[bi, first_needed:min(need_pages, lay.width)]
            need(need_pages <= lay.width and bool((row > 0).all()),
                 f"group {g.key}: sequence {bi} has keys on a page it does not hold")


def build_step_batch(entries: list, cache, device, pin: bool = True, check=None,
                     pad_to=None) -> StepBatch:
    """Pack ``entries`` (``SequenceInput``; pages already allocated) into a
    ``StepBatch`` on ``device``.  ``check(host array, layout)``: called on the packed
    metadata before it is copied (debug checks).  ``pad_to(StepShape)``: the number of token
    rows the step is to run with (its own or more); the rows beyond its own belong to one
    padding sequence (``fill_packed``), which the host-side lengths list like a sequence of
    that many new tokens: the attention works on its rows too (over page 0), so every row of
    every activation is a finite number and what the padding rows leave on page 0 is too (a
    key tile's masked keys may lie there: their values are multiplied by zero, which must
    not meet a NaN)."""
    shape = describe_step(entries, cache)
    group_list = list(cache.page_groups.values())
    rows = shape.t if pad_to is None else max(shape.t, int(pad_to(shape)))
    padded = rows > shape.t
    lay = PackedLayout(rows, len(shape.seqs) + (1 if padded else 0), len(shape.logit_index), shape.width,
                       len(group_list))
    host = np.zeros(lay.size, dtype=np.int32)
    num_patches = fill_packed(host, lay, shape, cache, group_list)
    if check is not None:
        check(host, lay)
    dev = torch.device(device)
    th = torch.from_numpy(host)
    if dev.type == "cuda":
        if pin:
            th = th.pin_memory()
        td = th.to(dev, non_blocking=True)
    else:
        td = th
    pad = [rows - shape.t] if padded else []
    batch = step_views(td, lay, group_list, shape.q_lens + pad, shape.kv_lens + pad,
                       shape.slots + ([0] if padded else []), shape.num_decode, shape.logit_rows,
                       shape.order)
    batch.num_patches = num_patches
    return batch
