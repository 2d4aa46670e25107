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


def _align(n: int, a: int = 4) -> int:
    return (n + a - 1) // a * a


def build_step_batch(entries: list, cache, device, pin: bool = True) -> StepBatch:
    """Pack ``entries`` (``SequenceInput``; pages already allocated) into a
    ``StepBatch`` on ``device``."""
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
    b = len(seqs)
    q_lens = [len(e.tokens) for e in seqs]
    kv_lens = [e.num_computed + len(e.tokens) for e in seqs]
    num_decode = sum(1 for q in q_lens if q == 1)
    t = sum(q_lens)

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
    r = len(logit_index)

    group_list = list(cache.page_groups.values())
    width = max(1, max(-(-kv // cache.page_size) for kv in kv_lens))

    # layout of the packed int32 array
    off = {}
    cur = 0
    for name, n in (("input_ids", t), ("positions", t), ("token_seq", t), ("cu_q_lens", b + 1),
                    ("seq_lens", b), ("state_slots", b), ("logit_indices", r)):
        off[name] = (cur, n)
        cur = _align(cur + n)
    for gi, g in enumerate(group_list):
        off[("bt", gi)] = (cur, b * width)
        cur = _align(cur + b * width)
        off[("sm", gi)] = (cur, t)
        cur = _align(cur + t)
    host = np.zeros(max(cur, 1), dtype=np.int32)

    def seg(name):
        s, n = off[name]
        return host[s:s + n]

    ids, pos, tseq = seg("input_ids"), seg("positions"), seg("token_seq")
    cu = seg("cu_q_lens")
    start = 0
    for bi, e in enumerate(seqs):
        q = q_lens[bi]
        ids[start:start + q] = e.tokens
        pos[start:start + q] = np.arange(e.num_computed, e.num_computed + q)
        tseq[start:start + q] = bi
        cu[bi + 1] = start + q
        start += q
    seg("seq_lens")[:] = kv_lens
    slots = [e.slot for e in seqs]
    seg("state_slots")[:] = slots
    seg("logit_indices")[:] = logit_index
    for gi, g in enumerate(group_list):
        seg(("bt", gi))[:] = cache.block_table(g, slots, width).reshape(-1)
        sm = seg(("sm", gi))
        start = 0
        for bi, e in enumerate(seqs):
            q = q_lens[bi]
            sm[start:start + q] = cache.slot_mapping(g, e.slot, e.num_computed, q)
            start += q

    dev = torch.device(device)
    th = torch.from_numpy(host)
    if dev.type == "cuda":
        if pin:
            th = th.pin_memory()
        td = th.to(dev, non_blocking=True)
    else:
        td = th

    def dseg(name):
        s, n = off[name]
        return td[s:s + n]

    groups = {}
    for gi, g in enumerate(group_list):
        groups[g.key] = AttentionMeta(
            block_table=dseg(("bt", gi)).view(b, width), slot_mapping=dseg(("sm", gi)),
            token_seq=dseg("token_seq"), positions=dseg("positions"), cu_q_lens=dseg("cu_q_lens"),
            seq_lens=dseg("seq_lens"), q_lens=q_lens, kv_lens=kv_lens, num_decode=num_decode)
    return StepBatch(
        num_tokens=t, num_seqs=b, num_decode=num_decode, num_logits=r,
        input_ids=dseg("input_ids"), positions=dseg("positions"), token_seq=dseg("token_seq"),
        cu_q_lens=dseg("cu_q_lens"), seq_lens=dseg("seq_lens"), state_slots=dseg("state_slots"),
        logit_indices=dseg("logit_indices"), q_lens=q_lens, kv_lens=kv_lens, slots=slots,
        groups=groups, logit_rows=logit_rows, order=order)
