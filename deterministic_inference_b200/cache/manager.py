"""Cache manager: paged keys and values with a block table per request, one page
pool per group of layers with the same need, and slots for per-request state of
fixed size.

The reference keeps token-granular slots (page size 1) in one LIFO stack shared
by all layers, a ``req_to_token`` row per request, and frees everything when a
request retires (sid/engine/kv_cache.py:22-93, sid/engine/scheduler.py:92-111).
Here:

* a page holds ``page_size`` tokens; page 0 of every pool is never handed out
  (block-table padding and skipped writes point at it);
* caches whose mixers have the same need (``spec.group_key()``: all keys, or a
  window of them, of the same head count and size) form a group with its own
  pool ``[caches, pages, 2, kv_heads, page_size, head_dim]``, its own free list
  (LIFO: the page freed last is handed out first) and its own block tables;
* a request holds one state slot from admission to its end; the slot indexes its
  block-table rows and the rows of every fixed-size state array
  ``[caches, max_reqs, *shape]``;
* pages go back to the free list when the request ends, and, in a window group,
  as soon as every position of the page is older than the window of the next
  query.

All bookkeeping is on the host; nothing here synchronises with the device.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import numpy as np
import torch

from ..parts.spec import PagedKVSpec, StateSpec

NULL_PAGE = 0


class CacheError(RuntimeError):
    pass


class OutOfPages(CacheError):
    pass


@dataclass
class CacheView:
    """What a mixer sees of the one cache its schedule entry names."""

    kv: Optional[torch.Tensor] = None            # [pages, 2, Hkv, page_size, D] of this cache
    page_size: int = 0
    slot_mapping: Optional[torch.Tensor] = None  # int32 [T]: page * page_size + offset
    attention_meta: object = None                # the group's AttentionMeta of this step
    state: Optional[torch.Tensor] = None         # [max_reqs, *shape] of this cache
    writes: bool = True


class PageGroup:
    """Pool, free list and per-request page lists of one group of caches."""

    def __init__(self, key, spec: PagedKVSpec, cache_ids: list[int], num_pages: int,
                 page_size: int, max_reqs: int):
        if num_pages < 2:
            raise CacheError("a page pool needs at least 2 pages (page 0 is never handed out)")
        self.key, self.spec, self.cache_ids = key, spec, list(cache_ids)
        self.num_pages, self.page_size = int(num_pages), int(page_size)
        self.window = spec.window
        # LIFO: pop() takes from the end; low page ids are handed out first at start
        self.free: list[int] = list(range(num_pages - 1, 0, -1))
        self.held: set[int] = set()
        self.pages: list[list[int]] = [[] for _ in range(max_reqs)]
        self.pool: Optional[torch.Tensor] = None

    @property
    def num_free(self) -> int:
        return len(self.free)

    def pages_needed(self, slot: int, total_len: int) -> int:
        have = len(self.pages[slot])
        want = -(-total_len // self.page_size)
        return max(0, want - have)

    def extend(self, slot: int, total_len: int) -> None:
        n = self.pages_needed(slot, total_len)
        if n > len(self.free):
            raise OutOfPages(f"group {self.key}: need {n} pages, {len(self.free)} free")
        for _ in range(n):
            p = self.free.pop()
            if p in self.held or p == NULL_PAGE:
                raise CacheError(f"free list handed out page {p} that is held")
            self.held.add(p)
            self.pages[slot].append(p)

    def _give_back(self, p: int) -> None:
        if p == NULL_PAGE:
            return
        if p not in self.held:
            raise CacheError(f"page {p} freed twice or never handed out")
        self.held.remove(p)
        self.free.append(p)

    def release_passed(self, slot: int, next_position: int) -> int:
        """Window groups: give back pages all of whose positions are older than
        the window of a query at ``next_position``.  Returns how many."""
        if self.window is None:
            return 0
        first_needed = next_position - self.window + 1
        n = 0
        pl = self.pages[slot]
        for i in range(len(pl)):
            if (i + 1) * self.page_size <= first_needed:
                if pl[i] != NULL_PAGE:
                    self._give_back(pl[i])
                    pl[i] = NULL_PAGE
                    n += 1
            else:
                break
        return n

    def release_all(self, slot: int) -> None:
        for p in self.pages[slot]:
            self._give_back(p)
        self.pages[slot] = []


class StateGroup:
    def __init__(self, key, spec: StateSpec, cache_ids: list[int]):
        self.key, self.spec, self.cache_ids = key, spec, list(cache_ids)
        self.array: Optional[torch.Tensor] = None


def _element_size(dtype: torch.dtype) -> int:
    return torch.empty(0, dtype=dtype).element_size()


def group_page_bytes(cache_specs: dict, page_size: int, dtype: torch.dtype) -> dict:
    """group key -> (spec, bytes of one page over all caches of the group), for the groups
    of paged caches among ``cache_specs`` (cache id -> need)."""
    count: dict = {}
    specs: dict = {}
    for spec in cache_specs.values():
        if isinstance(spec, PagedKVSpec):
            count[spec.group_key()] = count.get(spec.group_key(), 0) + 1
            specs[spec.group_key()] = spec
    item = _element_size(dtype)
    return {k: (specs[k], n * 2 * specs[k].num_kv_heads * page_size * specs[k].head_dim * item)
            for k, n in count.items()}


def pages_for_budget(cache_specs: dict, byte_budget: int, page_size: int, dtype: torch.dtype,
                     max_reqs: int, step_tokens: int) -> dict:
    """Pages per group (page 0 included) that ``byte_budget`` bytes pay for.  Groups that keep
    all keys get the same number of pages n, as many as fit.  A window group never needs more
    than what ``max_reqs`` requests can hold at a time (the window, a step's new tokens and
    two pages of rounding each), so it gets min(n, that) and the bytes saved go to the
    others."""
    groups = group_page_bytes(cache_specs, page_size, dtype)
    if not groups:
        return {}
    cap = {}
    for k, (spec, _) in groups.items():
        if spec.window is not None:
            cap[k] = 1 + max_reqs * (-(-(spec.window + step_tokens) // page_size) + 2)
    lo, hi = 2, max(2, byte_budget // min(b for _, b in groups.values()))
    def cost(n):
        return sum(min(n, cap.get(k, n)) * b for k, (_, b) in groups.items())
    if cost(lo) > byte_budget:
        raise CacheError(f"{byte_budget} bytes do not pay for two pages in every cache group "
                         f"({cost(lo)} bytes)")
    while lo < hi:                       # the largest n whose cost fits
        mid = (lo + hi + 1) // 2
        if cost(mid) <= byte_budget:
            lo = mid
        else:
            hi = mid - 1
    return {k: min(lo, cap.get(k, lo)) for k in groups}


class CacheManager:
    def __init__(self, cache_specs: dict, num_pages, page_size: int, max_reqs: int,
                 max_seq_len: int, dtype: torch.dtype = torch.bfloat16, device="cuda",
                 allocate_device: bool = True):
        """``num_pages``: pages of every group's pool (page 0 included), or a dict from
        group key to the pages of that group (``pages_for_budget``)."""
        self.page_size, self.max_reqs = int(page_size), int(max_reqs)
        self.max_seq_len = int(max_seq_len)
        self.max_blocks = -(-self.max_seq_len // self.page_size)
        self.dtype, self.device = dtype, torch.device(device)
        self.page_groups: dict[tuple, PageGroup] = {}
        self.state_groups: dict[tuple, StateGroup] = {}
        self._where: dict[int, tuple] = {}       # cache id -> (group, index in group)

        by_key: dict[tuple, list[int]] = {}
        specs: dict[tuple, object] = {}
        for cid in sorted(cache_specs):
            spec = cache_specs[cid]
            by_key.setdefault(spec.group_key(), []).append(cid)
            specs[spec.group_key()] = spec
        for key, cids in by_key.items():
            spec = specs[key]
            if isinstance(spec, PagedKVSpec):
                n = num_pages[key] if isinstance(num_pages, dict) else num_pages
                g = PageGroup(key, spec, cids, n, page_size, max_reqs)
                self.page_groups[key] = g
            elif isinstance(spec, StateSpec):
                g = StateGroup(key, spec, cids)
                self.state_groups[key] = g
            else:
                raise CacheError(f"cache {cids}: unknown need {spec!r}")
            for i, cid in enumerate(cids):
                self._where[cid] = (g, i)

        # state slots: slot 0 is never handed out (padding rows of a batch use it)
        self.free_slots: list[int] = list(range(max_reqs - 1, 0, -1))
        self.live_slots: set[int] = set()
        self.fresh_slots: list[int] = []     # handed out since the last step: state to be zeroed
        if allocate_device:
            self.allocate_device_memory()

    # ---- device memory --------------------------------------------------------

    def bytes_per_page(self) -> int:
        """Bytes of one page over all groups and caches (for sizing the pool)."""
        item = _element_size(self.dtype)
        return sum(len(g.cache_ids) * 2 * g.spec.num_kv_heads * g.page_size * g.spec.head_dim * item
                   for g in self.page_groups.values())

    def allocate_device_memory(self) -> None:
        for g in self.page_groups.values():
            g.pool = torch.zeros(len(g.cache_ids), g.num_pages, 2, g.spec.num_kv_heads, g.page_size,
                                 g.spec.head_dim, dtype=self.dtype, device=self.device)
        for g in self.state_groups.values():
            dt = getattr(torch, g.spec.dtype)
            g.array = torch.zeros(len(g.cache_ids), self.max_reqs, *g.spec.shape, dtype=dt,
                                  device=self.device)

    # ---- state slots ------------------------------------------------------------

    @property
    def num_free_slots(self) -> int:
        return len(self.free_slots)

    def allocate_slot(self) -> int:
        if not self.free_slots:
            raise CacheError("no free state slot")
        s = self.free_slots.pop()
        if s in self.live_slots:
            raise CacheError(f"state slot {s} handed out twice")
        self.live_slots.add(s)
        self.fresh_slots.append(s)
        return s

    def release_slot(self, slot: int) -> None:
        """End of a request (or its preemption): every page of every group and
        the slot itself go back."""
        if slot not in self.live_slots:
            raise CacheError(f"state slot {slot} released twice or never handed out")
        for g in self.page_groups.values():
            g.release_all(slot)
        self.live_slots.remove(slot)
        self.free_slots.append(slot)
        if slot in self.fresh_slots:
            self.fresh_slots.remove(slot)

    def take_fresh_slots(self) -> list[int]:
        out, self.fresh_slots = self.fresh_slots, []
        return out

    def reset_fresh_state(self) -> None:
        """Zero the state rows of slots handed out since the last call."""
        fresh = self.take_fresh_slots()
        if fresh and self.state_groups:
            idx = torch.tensor(fresh, dtype=torch.long, device=self.device)
            for g in self.state_groups.values():
                if g.array is not None:
                    g.array[:, idx] = 0

    # ---- pages ---------------------------------------------------------------------

    def num_free_pages(self) -> int:
        """Free pages of the tightest group (a request needs pages in each)."""
        if not self.page_groups:
            return 1 << 30
        return min(g.num_free for g in self.page_groups.values())

    def usable_pages(self) -> int:
        """Pages a request can ever hold in the groups that keep all keys (they bound how
        long a request may grow; a window group gives pages back as the window moves)."""
        full = [g.num_pages - 1 for g in self.page_groups.values() if g.window is None]
        if not full:
            return 1 << 30
        return min(full)

    def can_allocate(self, slot: Optional[int], total_len: int) -> bool:
        """Whether every group can cover positions < total_len of the request in
        ``slot`` (None: a request that holds nothing yet)."""
        for g in self.page_groups.values():
            need = g.pages_needed(slot, total_len) if slot is not None \
                else -(-total_len // g.page_size)
            if need > g.num_free:
                return False
        return True

    def allocate(self, slot: int, total_len: int) -> None:
        """Make every group cover positions < total_len for ``slot``; all or
        nothing (raises ``OutOfPages`` and leaves the request as it was)."""
        if slot not in self.live_slots:
            raise CacheError(f"allocate for slot {slot} that is not live")
        if total_len > self.max_seq_len:
            raise CacheError(f"sequence of {total_len} tokens exceeds max_seq_len {self.max_seq_len}")
        if not self.can_allocate(slot, total_len):
            raise OutOfPages(f"not enough free pages for {total_len} tokens in slot {slot}")
        for g in self.page_groups.values():
            g.extend(slot, total_len)

    def release_passed(self, slot: int, next_position: int) -> int:
        return sum(g.release_passed(slot, next_position) for g in self.page_groups.values())

    # ---- what a step needs ------------------------------------------------------------

    def block_table(self, group: PageGroup, slots: list[int], width: int) -> np.ndarray:
        out = np.zeros((len(slots), width), dtype=np.int32)
        for r, s in enumerate(slots):
            pl = group.pages[s]
            n = min(len(pl), width)
            out[r, :n] = pl[:n]
        return out

    def slot_mapping(self, group: PageGroup, slot: int, start: int, n: int) -> np.ndarray:
        """Cache slots (page * page_size + offset) of positions start .. start+n-1."""
        pos = np.arange(start, start + n, dtype=np.int64)
        pl = np.asarray(group.pages[slot], dtype=np.int64)
        pages = pl[pos // group.page_size]
        if (pages == NULL_PAGE).any():
            raise CacheError(f"slot {slot}: positions {start}..{start + n - 1} are not covered by pages")
        return (pages * group.page_size + pos % group.page_size).astype(np.int32)

    def group_of(self, cache_id: int):
        return self._where[cache_id][0]

    def view(self, cache_id: int, step, writes: bool = True) -> CacheView:
        g, i = self._where[cache_id]
        if isinstance(g, PageGroup):
            gb = step.groups[g.key]
            return CacheView(kv=g.pool[i] if g.pool is not None else None, page_size=g.page_size,
                             slot_mapping=gb.slot_mapping, attention_meta=gb, writes=writes)
        return CacheView(state=g.array[i] if g.array is not None else None, writes=writes)

    # ---- checks ---------------------------------------------------------------------------

    def check_invariants(self) -> None:
        """No page lost, held twice or free and held at once; slots likewise."""
        for g in self.page_groups.values():
            free = list(g.free)
            if len(set(free)) != len(free):
                raise CacheError(f"group {g.key}: a page is on the free list twice")
            owned: list[int] = []
            for s, pl in enumerate(g.pages):
                live = [p for p in pl if p != NULL_PAGE]
                if live and s not in self.live_slots:
                    raise CacheError(f"group {g.key}: slot {s} holds pages but is not live")
                owned.extend(live)
            if len(set(owned)) != len(owned):
                raise CacheError(f"group {g.key}: a page is held by two requests")
            if set(owned) != g.held:
                raise CacheError(f"group {g.key}: held set and page lists disagree")
            if set(owned) & set(free):
                raise CacheError(f"group {g.key}: a page is free and held at once")
            if set(owned) | set(free) != set(range(1, g.num_pages)):
                raise CacheError(f"group {g.key}: a page is lost")
        if set(self.free_slots) & self.live_slots:
            raise CacheError("a state slot is free and live at once")
        if set(self.free_slots) | self.live_slots != set(range(1, self.max_reqs)):
            raise CacheError("a state slot is lost")
