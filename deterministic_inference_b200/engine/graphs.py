"""CUDA-graph replay of pure-decode steps (every sequence brings one token and
wants its logits).

A decode step of a small model is bound by launch latency, not by the GPU.  For
a bucket of batch size and block-table width the step function is captured once:
its kernels read the step's integer metadata from ONE static device array, so a
later step only copies its packed metadata into that array (one host-to-device
copy from pinned memory) and replays the graph.  Batches are padded to the
bucket with sequences that live on the cache's page 0 and state slot 0, which no
request owns.  Grid sizes that depend on sequence lengths are captured for the
longest sequence the block-table width allows; blocks beyond a sequence's real
length exit at once.
"""

from __future__ import annotations

import numpy as np
import torch

import contextlib
import dataclasses
import gc
import time
from collections import OrderedDict

from .batch import PackedLayout, SequenceInput, describe_step, fill_packed, step_views


@contextlib.contextmanager
def _no_collection():
    """No cyclic garbage collection while a graph is captured: a collected object that
    owns device memory or another graph would call into CUDA in the middle of the
    capture and invalidate it.  (The collector is only switched off, not run first: a
    full collection takes as long as the capture itself, some 30 ms.)"""
    was = gc.isenabled()
    gc.disable()
    try:
        yield
    finally:
        if was:
            gc.enable()


def _bucket(n: int, smallest: int = 1) -> int:
    b = smallest
    while b < n:
        b *= 2
    return b


class _Captured:
    """A captured step.  ``batch`` is kept because the captured kernels use what it
    holds: the views of ``static_meta`` and the scratch memory kernels attached to
    it during the warm-up runs (the decode attention's split workspace)."""

    def __init__(self, graph, static_meta, host_meta, layout, logits, batch):
        self.graph, self.static_meta, self.host_meta = graph, static_meta, host_meta
        self.layout, self.logits, self.batch = layout, logits, batch
        self.uploaded = torch.cuda.Event()
        self.check = None        # debug check of the packed metadata (host array, layout)

    def upload(self, fill, num_prev: int = 0) -> object:
        """Fill the pinned metadata (``fill(array)``) and copy it to the device.  The
        pinned array is written again only after the copy before has run: a caller may
        issue steps faster than the GPU takes them."""
        self.uploaded.synchronize()
        result = fill(self.host_meta.numpy())
        if self.check is not None:
            self.check(self.host_meta.numpy(), self.layout, num_prev)
        self.static_meta.copy_(self.host_meta, non_blocking=True)
        self.uploaded.record()
        return result


class DecodeGraphs:
    def __init__(self, model, cache, device, max_batch: int = 256, min_width: int = 8):
        # the model, the cache and the device, not the runner that owns this object: a
        # cycle would leave captured graphs to the garbage collector
        self.model, self.cache, self.device = model, cache, device
        self.max_batch = max_batch
        self.min_width = min_width
        self.graphs: dict[tuple, _Captured] = {}
        self.group_list = list(self.cache.page_groups.values())
        self.replays = 0
        self.captures = 0
        self.capture_seconds = 0.0
        self.kernels_per_graph: dict[tuple, int] = {}
        self.kernels_replayed = 0          # kernels inside the graphs replayed so far
        self.check = None                  # debug check of every step's packed metadata
        # one memory pool for all graphs of this object: only one of them runs at a time,
        # and what a replay leaves (its logits) is read before the next replay is issued
        self.pool = torch.cuda.graph_pool_handle() if torch.cuda.is_available() else None

    def usable(self, entries) -> bool:
        """Pure-decode steps only; and not while a part keeps per-request state: the
        capture runs the model twice as a warm-up, which would advance that state, and
        such a part may read its slots on the host."""
        return (not self.cache.state_groups and 0 < len(entries) <= self.max_batch
                and all(len(e.tokens) == 1 and list(e.want) == [0] for e in entries))

    # ---- capture ---------------------------------------------------------------

    def _key(self, shape) -> tuple:
        # block-table width: powers of two up to 32 pages, then multiples of 32 (grids
        # sized for the width's longest sequence should not be mostly empty)
        width = shape.width
        wb = _bucket(width, self.min_width) if width <= 32 else -(-width // 32) * 32
        return (_bucket(len(shape.seqs)), min(wb, self.cache.max_blocks))

    def _capture(self, key: tuple, shape) -> _Captured:
        t0 = time.perf_counter()
        cap = self._capture_timed(key, shape)
        self.captures += 1
        self.capture_seconds += time.perf_counter() - t0
        return cap

    def _capture_timed(self, key: tuple, shape) -> _Captured:
        bb, w = key
        dev = self.device
        lay = PackedLayout(bb, bb, bb, w, len(self.group_list))
        host = torch.zeros(lay.size, dtype=torch.int32).pin_memory()
        static = torch.zeros(lay.size, dtype=torch.int32, device=dev)
        upper = w * self.cache.page_size
        batch = step_views(static, lay, self.group_list, [1] * bb, [upper] * bb, [0] * bb, bb,
                           [[i] for i in range(bb)], list(range(bb)))
        fill_packed(host.numpy(), lay, shape, self.cache, self.group_list)
        static.copy_(host, non_blocking=True)
        # warm up on a side stream (library handles, lazy module loading), then capture
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for _ in range(2):
                self.model.forward(batch, self.cache)
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        from ..kernels import ops
        ops.check_kernel_status()        # the warm-up launched every kernel of the step
        n0 = ops.launch_count
        graph = torch.cuda.CUDAGraph()
        with _no_collection(), torch.cuda.graph(graph, pool=self.pool):
            logits = self.model.forward(batch, self.cache)
        self.kernels_per_graph[key] = ops.launch_count - n0
        cap = _Captured(graph, static, host, lay, logits, batch)
        cap.check = self.check
        self.graphs[key] = cap
        return cap

    # ---- replay -------------------------------------------------------------------

    @torch.inference_mode()
    def run(self, entries, prev_tokens=None):
        """(logits [B, V], StepBatch) for a pure-decode step whose pages are allocated
        already.  The logits are a view of the graph's own buffer: they hold until the
        next replay of a decode graph."""
        cache = self.cache
        shape = describe_step(entries, cache)
        key = self._key(shape)
        cap = self.graphs.get(key)
        if cap is None:
            cap = self._capture(key, shape)
        num_patches = cap.upload(
            lambda host: fill_packed(host, cap.layout, shape, cache, self.group_list),
            0 if prev_tokens is None else int(prev_tokens.shape[0]))
        if num_patches:
            from ..kernels import ops
            ops.patch_token_ids(cap.batch.input_ids, cap.batch.patch_dst, cap.batch.patch_src,
                                prev_tokens)
        cap.graph.replay()
        self.replays += 1
        self.kernels_replayed += self.kernels_per_graph.get(key, 0)
        batch = dataclasses.replace(cap.batch, logit_rows=shape.logit_rows, order=shape.order,
                                    slots=shape.slots)
        batch.num_patches = num_patches
        return cap.logits[:len(entries)], batch


def token_bucket(q: int) -> tuple:
    """(bucket, smallest count of the bucket) for a sequence that brings ``q`` >= 2 tokens
    to a step: counts are rounded up to a multiple of a sixteenth of the power of two at or
    below them (16 at least), so a bucket's graph runs 6 % more rows than the step has at
    worst and about 3 % on average, with 16 buckets to an octave."""
    step = max(16, (1 << (q.bit_length() - 1)) // 16)
    b = -(-q // step) * step
    return b, max(2, b - step + 1)


class StepGraphs:
    """CUDA-graph replay of steps that are no pure decode steps: portions of prompts, whole
    prompts, and those beside decoded tokens.  A small model's step of 2,048 prompt tokens
    is a few hundred launches that the host issues barely faster than the GPU runs them.

    A graph is captured for a BUCKET of step shapes: the number of one-token sequences
    rounded up to a power of two (the step is filled up with padding entries on state slot 0,
    one token and one dropped logits row each, as the decode graphs' batches are), the same
    number of prompt portions, each one's token count rounded up (``token_bucket``), the same
    number of wanted logits rows, block tables of the same bucket of width.  The step's real counts reach the kernels through the packed metadata
    on the device; what the host knows when it captures (grids, the attention's list of query
    tiles) is sized for the bucket's upper bounds, and a query tile past a sequence's real
    tokens leaves at once.  The rows that a step does not fill belong to a padding sequence
    on page 0 and state slot 0 (``fill_packed``) and follow the step's own rows; every
    kernel works row by row or takes a row's sequence from the metadata, so they reach no
    request's result (they are worked on like a request's rows, so that they hold finite
    numbers and leave such on page 0).  A bucket is captured when it shows up the third time; the least
    recently used graph goes when there are more than ``max_graphs`` (they share one memory
    pool).  A capture costs two runs of the step and the graph's instantiation, and a replay only wins where the host
    issues the step's launches no faster than the GPU runs them: so a bucket's launched steps
    are timed (host time to issue them, device time between two events), and a bucket whose
    launches took the host less than ``host_bound_share`` of the device's time is captured
    only when it has shown up ``patient_repeats`` times: there a replay saves the few
    microseconds between two launches only (4-5 % of a step of 2,048 tokens at 8B layer
    sizes), which pays for the capture after a hundred replays or so.  Not used while the cache holds per-request state of a part (a part may read its
    slots on the host)."""

    def __init__(self, model, cache, device, max_graphs: int = 64, min_repeats: int = 3,
                 min_width: int = 8, host_bound_share: float = 0.5, patient_repeats: int = 16):
        # the model, the cache and the device, not the runner that owns this object: a
        # cycle would leave captured graphs to the garbage collector, which may then
        # destroy one in the middle of another capture
        self.model, self.cache, self.device = model, cache, device
        self.max_graphs, self.min_repeats, self.min_width = max_graphs, min_repeats, min_width
        self.host_bound_share, self.patient_repeats = host_bound_share, patient_repeats
        self.graphs: "OrderedDict[tuple, _Captured]" = OrderedDict()
        self.seen: dict = {}
        self.timings: dict = {}            # bucket -> (host seconds, event, event) of its last launched step
        self.device_bound: set = set()     # buckets whose launched steps the device, not the host, bounds
        self._launching = None             # the bucket of the step that run() just declined
        self.group_list = list(self.cache.page_groups.values())
        self.replays = 0
        self.captures = 0
        self.capture_seconds = 0.0
        self.kernels_per_graph: dict[tuple, int] = {}
        self.kernels_replayed = 0
        self.check = None                  # debug check of every step's packed metadata
        # one memory pool for all graphs (their activations never live at the same time;
        # a replay's logits are copied out before the next replay)
        self.pool = torch.cuda.graph_pool_handle() if torch.cuda.is_available() else None

    def _width_bucket(self, width: int) -> int:
        wb = _bucket(width, self.min_width) if width <= 32 else -(-width // 32) * 32
        return min(wb, self.cache.max_blocks)

    @staticmethod
    def padded_tokens(shape) -> int:
        """The token rows a step of this shape runs with, replayed or launched: its one-token
        sequences rounded up to a power of two, plus the sum of the other sequences' buckets.
        A step that is launched kernel by kernel (its bucket has not come three times yet)
        runs with the same number of rows as the graph will, so that a library's choice of
        algorithm by the row count, and with it a token's bits, does not depend on how often
        a bucket has been seen."""
        nd = sum(1 for q in shape.q_lens if q == 1)
        return (_bucket(nd) if nd else 0) + sum(token_bucket(q)[0] for q in shape.q_lens if q != 1)

    def run(self, entries, prev_tokens=None):
        """(logits, StepBatch) like ``ModelRunner.step``, or None if this step is to be
        run launch by launch.  The pages of the entries are allocated already."""
        if self.cache.state_groups:
            return None
        n_own = len(entries)
        nd = sum(1 for e in entries if len(e.tokens) == 1)
        if nd and _bucket(nd) > nd:      # fill the bucket of one-token sequences with padding entries
            entries = list(entries) + [SequenceInput(0, [0], 0, [0])] * (_bucket(nd) - nd)
        shape = describe_step(entries, self.cache)
        n_fill = len(entries) - n_own
        wb = self._width_bucket(shape.width)
        if wb < shape.width:
            return None
        buckets = [(1, 1) if q == 1 else token_bucket(q) for q in shape.q_lens]
        key = (tuple(b for b, _ in buckets), len(shape.logit_index), wb)
        cap = self.graphs.get(key)
        self._launching = None
        if cap is None:
            n = self.seen.get(key, 0) + 1
            if len(self.seen) > 4096:
                self.seen.clear()
                self.timings.clear()
                self.device_bound.clear()
            self.seen[key] = n
            if key in self.device_bound:
                if n < self.patient_repeats:
                    return None
            elif n < self.min_repeats or not self._host_bound(key):
                self._launching = key if key not in self.device_bound else None
                return None
            t0 = time.perf_counter()
            cap = self._capture(key, shape, buckets, wb)
            self.capture_seconds += time.perf_counter() - t0
        else:
            self.graphs.move_to_end(key)
        num_patches = cap.upload(
            lambda host: fill_packed(host, cap.layout, shape, self.cache, self.group_list),
            0 if prev_tokens is None else int(prev_tokens.shape[0]))
        if num_patches:
            from ..kernels import ops
            ops.patch_token_ids(cap.batch.input_ids, cap.batch.patch_dst, cap.batch.patch_src,
                                prev_tokens)
        cap.graph.replay()
        self.replays += 1
        self.kernels_replayed += self.kernels_per_graph.get(key, 0)
        # the caller owns what it gets (the graph's own logits are overwritten by its next
        # replay) and sees its own entries only: the padding entries' rows lie in one run, behind
        # those of its one-token sequences and before those of its prompt portions
        if n_fill:
            a = shape.logit_rows[n_own][0]       # the padding entries' rows: a .. a + n_fill - 1
            logits = torch.cat([cap.logits[:a], cap.logits[a + n_fill:]])
            logit_rows = [[r if r < a else r - n_fill for r in rows] for rows in shape.logit_rows[:n_own]]
            order = [i for i in shape.order if i < n_own]
        else:
            logits, logit_rows, order = cap.logits.clone(), shape.logit_rows, shape.order
        batch = dataclasses.replace(cap.batch, logit_rows=logit_rows, order=order, slots=shape.slots)
        batch.num_patches = num_patches
        return logits, batch

    def launched(self, host_seconds: float, start, end) -> None:
        """The runner's report on the step that ``run`` just declined: the host's time to issue
        its launches and the CUDA events recorded around them."""
        if self._launching is not None:
            self.timings[self._launching] = (host_seconds, start, end)
            self._launching = None

    def _host_bound(self, key) -> bool:
        """Whether the bucket's last launched step kept the GPU waiting for the host; False
        while that step has not finished (the host is not made to wait for it: the bucket is
        asked about again the next time).  A bucket found to be bound by the device is
        remembered and not timed again."""
        t = self.timings.get(key)
        if t is None or not t[2].query():
            return False
        host_s, start, end = t
        device_s = start.elapsed_time(end) / 1e3
        if host_s >= self.host_bound_share * device_s:
            return True
        self.device_bound.add(key)
        self.timings.pop(key, None)
        return False

    def _capture(self, key: tuple, shape, buckets: list, wb: int) -> _Captured:
        dev = self.device
        b = len(shape.seqs)
        q_upper = [qb for qb, _ in buckets]
        # one more sequence than the step has: the padding sequence that owns the rows a
        # step of this bucket does not fill
        lay = PackedLayout(sum(q_upper), b + 1, len(shape.logit_index), wb, len(self.group_list))
        host = torch.zeros(lay.size, dtype=torch.int32).pin_memory()
        static = torch.zeros(lay.size, dtype=torch.int32, device=dev)
        # What kernels size their grids and lists for: every sequence as long as the block
        # table's width allows, and as many tokens before a portion as the shortest portion
        # of its bucket would leave of that (the lists take key counts minus new tokens as
        # the tokens before a portion).
        upper = wb * self.cache.page_size
        kv_upper = [upper + qb - lo for qb, lo in buckets]
        # the padding sequence has the rows that the sequences of a step leave: as many as
        # the shortest of each bucket would leave, at most.  The attention works on them
        # too (over page 0), so that every row of every activation is a finite number.
        pad_upper = sum(qb - lo for qb, lo in buckets)
        batch = step_views(static, lay, self.group_list, q_upper + [pad_upper], kv_upper + [pad_upper],
                           list(shape.slots) + [0], shape.num_decode, shape.logit_rows, shape.order)
        fill_packed(host.numpy(), lay, shape, self.cache, self.group_list)
        static.copy_(host, non_blocking=True)
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            # one run before the capture: what the kernels attach to this batch (tile lists,
            # scratch) is made outside it; the bucket's launched steps have loaded every kernel
            self.model.forward(batch, self.cache)
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        from ..kernels import ops
        ops.check_kernel_status()        # the warm-up launched every kernel of the step
        while len(self.graphs) >= self.max_graphs:      # before the capture, not inside it
            self.graphs.popitem(last=False)
        n0 = ops.launch_count
        graph = torch.cuda.CUDAGraph()
        with _no_collection(), torch.cuda.graph(graph, pool=self.pool):
            logits = self.model.forward(batch, self.cache)
        self.kernels_per_graph[key] = ops.launch_count - n0
        cap = _Captured(graph, static, host, lay, logits, batch)
        cap.check = self.check
        self.graphs[key] = cap
        self.captures += 1
        return cap
