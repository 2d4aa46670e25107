"""Helpers for attention tests: put dense keys/values of several sequences into a
paged cache with shuffled, non-contiguous pages, and build the step metadata for
a given cut (how many cached tokens, how many new ones per sequence)."""

from __future__ import annotations

import torch

from deterministic_inference_b200.engine.batch import AttentionMeta


def dense_reference(q, k, v, scale, q_positions, window=None):
    """float32 attention of queries at absolute ``q_positions`` over keys 0..p of
    one sequence.  q [n, Hq, D]; k, v [L, Hkv, D] (tests/conftest.py:11-32 of the
    reference, with the causal offset written as absolute positions)."""
    n, hq, d = q.shape
    hkv = k.shape[1]
    g = hq // hkv
    qf, kf, vf = q.double(), k.double(), v.double()
    out = torch.empty(n, hq, d, dtype=torch.float64, device=q.device)
    keys = torch.arange(k.shape[0], device=q.device)
    for i, p in enumerate(q_positions):
        vis = keys <= p
        if window:
            vis &= keys > p - window
        for h in range(hq):
            s = (kf[:, h // g] @ qf[i, h]) * scale
            s = s.masked_fill(~vis, float("-inf"))
            out[i, h] = torch.softmax(s, -1) @ vf[:, h // g]
    return out.float()


class PagedCase:
    """Several sequences with dense k/v, stored in one paged cache layer."""

    def __init__(self, lens, hkv, d, page_size, dtype, device="cuda", seed=0, extra_pages=7,
                 k=None, v=None):
        g = torch.Generator(device="cpu").manual_seed(seed)
        self.lens, self.page_size, self.hkv, self.d = list(lens), page_size, hkv, d
        self.k = k or [torch.randn(n, hkv, d, generator=g).to(device=device, dtype=dtype) for n in lens]
        self.v = v or [torch.randn(n, hkv, d, generator=g).to(device=device, dtype=dtype) for n in lens]
        pages_per = [-(-n // page_size) for n in lens]
        total = sum(pages_per) + extra_pages + 1
        perm = (torch.randperm(total - 1, generator=g) + 1).tolist()     # page 0 stays unused
        self.tables = []
        self.cache = torch.zeros(total, 2, hkv, page_size, d, dtype=dtype, device=device)
        # poison unused memory so that a read outside a sequence's pages shows
        self.cache.fill_(1000.0)
        for s, n in enumerate(lens):
            pl = [perm.pop() for _ in range(pages_per[s])]
            self.tables.append(pl)
            pos = torch.arange(n, device=device)
            pidx = torch.tensor(pl, device=device)[pos // page_size]
            self.cache[pidx, 0, :, pos % page_size] = self.k[s]
            self.cache[pidx, 1, :, pos % page_size] = self.v[s]
        self.device = device

    def meta(self, seqs, q_ranges):
        """``seqs``: indices of the sequences in the batch; ``q_ranges``: for each,
        (first new position, number of new tokens).  Sequences with one token must
        come first (the engine's batch order)."""
        width = max(len(self.tables[s]) for s in seqs)
        bt = torch.zeros(len(seqs), width, dtype=torch.int32)
        token_seq, positions, cu, kv_lens, q_lens = [], [], [0], [], []
        for b, (s, (start, n)) in enumerate(zip(seqs, q_ranges)):
            bt[b, :len(self.tables[s])] = torch.tensor(self.tables[s], dtype=torch.int32)
            token_seq += [b] * n
            positions += list(range(start, start + n))
            cu.append(cu[-1] + n)
            kv_lens.append(start + n)
            q_lens.append(n)
        dev = self.device
        i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
        nd = 0
        for n in q_lens:
            if n == 1:
                nd += 1
            else:
                break
        assert all(n > 1 for n in q_lens[nd:]), "one-token sequences must come first"
        return AttentionMeta(block_table=bt.to(dev), slot_mapping=i32([0] * len(token_seq)),
                             token_seq=i32(token_seq), positions=i32(positions), cu_q_lens=i32(cu),
                             seq_lens=i32(kv_lens), q_lens=q_lens, kv_lens=kv_lens, num_decode=nd)
