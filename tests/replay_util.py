"""Drives ``bin/trace_run`` as a user would (a subprocess, steps on its standard
input, ``done <step>`` awaited before the next step) and builds the cuttings of
a set of requests: whole, last 32 tokens one by one, portions of changing size,
and mixed with other requests in a pool so small that pages are used again."""

from __future__ import annotations

import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent.parent
TRACE_RUN = ROOT / "bin" / "trace_run"


def round_up(n, m):
    return -(-n // m) * m


class Trace:
    """Steps plus, for every written row, which (request, position) it is."""

    def __init__(self):
        self.steps: list[dict] = []
        self.rows: dict[int, list] = {}      # step -> [(request key, position)]
        self.peak_tokens = 0                  # most tokens live at a time, each rounded up to 64
        self._live: dict = {}

    def add_step(self, entries, end=()):
        """entries: [(key, first position, tokens, want places)]"""
        no = len(self.steps)
        rec = {"step": no, "entries": [], "end": [str(k) for k in end]}
        rows = []
        for key, start, toks, want in entries:
            rec["entries"].append({"id": str(key), "tokens": list(map(int, toks)), "want": list(want)})
            rows += [(key, start + w) for w in want]
            self._live[key] = start + len(toks)
        self.peak_tokens = max(self.peak_tokens, sum(round_up(n, 64) for n in self._live.values()))
        for k in end:
            self._live.pop(k, None)
        self.steps.append(rec)
        if rows:
            self.rows[no] = rows
        return no


def whole(trace, requests, prefix=""):
    for i, toks in enumerate(requests):
        k = f"{prefix}w{i}"
        trace.add_step([(k, 0, toks, list(range(len(toks))))], end=[k])


def last_one_by_one(trace, requests, tail=32, prefix=""):
    for i, toks in enumerate(requests):
        k = f"{prefix}t{i}"
        head = max(1, len(toks) - tail)
        if head == len(toks):
            trace.add_step([(k, 0, toks, list(range(len(toks))))], end=[k])
            continue
        trace.add_step([(k, 0, toks[:head], list(range(head)))])
        for p in range(head, len(toks)):
            trace.add_step([(k, p, toks[p:p + 1], [0])], end=[k] if p == len(toks) - 1 else [])


def portions(trace, requests, sizes=(13, 7, 2, 5, 2, 31, 3, 2, 64, 2), prefix=""):
    for i, toks in enumerate(requests):
        k = f"{prefix}p{i}"
        c, j = 0, i
        while c < len(toks):
            n = min(sizes[j % len(sizes)], len(toks) - c)
            if len(toks) - c - n == 1:     # never leave a single token for a "portion"
                n += 1
            j += 1
            last = c + n == len(toks)
            trace.add_step([(k, c, toks[c:c + n], list(range(n)))], end=[k] if last else [])
            c += n


def lockstep(trace, requests, portion=96, tail=8, prefix=""):
    """All requests (of one length) live at once and cut alike: every step brings the same
    portion of each, then single tokens, so the same step shapes come again and again (a
    step function that replays captured graphs of repeated shapes does so here)."""
    n = len(requests[0])
    assert all(len(r) == n for r in requests)
    keys = [f"{prefix}l{i}" for i in range(len(requests))]
    c = 0
    while c < n:
        left = n - c
        q = 1 if left <= tail else min(portion, left - tail)
        last = c + q == n
        trace.add_step([(k, c, r[c:c + q], list(range(q))) for k, r in zip(keys, requests)],
                       end=keys if last else [])
        c += q


def mixed(trace, requests, max_live=4, sizes=(11, 2, 17, 5, 2, 29, 3), tail=6, prefix=""):
    """Up to ``max_live`` requests at a time: each live request brings a portion
    (the last ``tail`` tokens one by one, like decoding), some steps leave a
    request out; finished requests end and new ones take over their pages."""
    waiting = list(enumerate(requests))
    live = []       # [key, tokens, computed]
    step = 0
    while waiting or live:
        while waiting and len(live) < max_live:
            i, toks = waiting.pop(0)
            live.append([f"{prefix}m{i}", toks, 0])
        entries, ended = [], []
        for li, item in enumerate(live):
            k, toks, c = item
            if (step + li) % 5 == 4 and len(live) > 1:
                continue                              # left out of this step, goes on later
            left = len(toks) - c
            n = 1 if left <= tail else min(sizes[(step + li) % len(sizes)], left - tail)
            entries.append((k, c, toks[c:c + n], list(range(n))))
            item[2] = c + n
            if item[2] == len(toks):
                ended.append(k)
        if entries:
            trace.add_step(entries, end=ended)
        live = [it for it in live if it[0] not in ended]
        step += 1


def run_trace(model_dir, dtype, trace, out_dir, max_tokens=None, page_size=16, timeout=900,
              user=None, cuda_graphs=False, extra_env=None):
    """Run the trace through bin/trace_run; returns {step: float32 array [wanted, V]}."""
    out_dir = Path(out_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    cmd = [sys.executable, str(TRACE_RUN), "--model", str(model_dir), "--dtype", dtype, "--out",
           str(out_dir), "--max-tokens", str(max_tokens or trace.peak_tokens),
           "--page-size", str(page_size)]
    if cuda_graphs:
        cmd.append("--cuda-graphs")
    env = dict(os.environ)
    env.update(extra_env or {})
    proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, env=env)
    try:
        for rec in trace.steps:
            proc.stdin.write(json.dumps(rec) + "\n")
            proc.stdin.flush()
            while True:
                line = proc.stdout.readline()
                if not line:
                    raise RuntimeError(f"trace_run ended at step {rec['step']} (exit {proc.wait()})")
                if line.strip() == f"done {rec['step']}":
                    break
        proc.stdin.close()
        code = proc.wait(timeout=timeout)
    finally:
        if proc.poll() is None:
            proc.kill()
    if code != 0:
        raise RuntimeError(f"trace_run exited with {code}")
    return out_dir


def read_rows(out_dir, trace, vocab):
    """{(request key, position): float32 tensor [V]} of everything the trace wrote."""
    got = {}
    for no, rows in trace.rows.items():
        arr = np.fromfile(Path(out_dir) / f"{no}.f32", dtype="<f4")
        assert arr.size == len(rows) * vocab, (no, arr.size, len(rows), vocab)
        arr = torch.from_numpy(arr.reshape(len(rows), vocab).copy())
        for r, key in enumerate(rows):
            got[key] = arr[r]
    return got
