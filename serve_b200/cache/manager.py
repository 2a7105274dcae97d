"""The cache manager: paged keys/values with per-request block tables, and state slots.

Layout. Every execution of a mixer that asked for pages owns a pair of device
tensors K, V of shape [num_pages, kv_heads, page_size, head_dim]
(the tokens of one kv head lie together inside a page, so attention reads
contiguous runs of page_size rows). Executions
with the same geometry and window form a *group*: one pool of page ids and one
block table per request serve all of them (page id p means page p in every
tensor of the group), as one id serves every layer in the reference
(serve/model.py:176-182). Groups with other needs (other head sizes, a window)
have pools and tables of their own. The reference's table is
[max_batch, kv_heads, blocks] with a page per kv head
(serve/kv_cache_paged.py:24-26); here a page holds all kv heads of its tokens,
so the table is [slot, block].

A request holds one *slot* while it lives: a row of every group's block table,
and a row of every fixed-size state tensor [max_slots, ...] that a mixer asked
for (zeroed when the slot is handed out). Llama asks for none.

Pages are given back when a request closes, and earlier when a group has a
window and the request has moved past a page. Block tables are kept on the
host; a step uploads the rows it uses (the reference reads them back from the
device to free them, kv_cache_paged.py:72).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import numpy as np

from ..parts.base import CacheNeed
from .pages import OutOfPages, PagePool


class NoFreeSlot(RuntimeError):
    pass


@dataclass
class CacheView:
    """What one execution of a mixer sees of the cache."""

    group: int                 # index into StepContext.block_tables
    k: object                  # [num_pages, kv_heads, page_size, head_dim] or None
    v: object
    page_size: int
    writes: bool               # False: reads the cache another execution wrote
    state: object = None       # [max_slots, *state_shape] float32 or None
    window: Optional[int] = None


@dataclass
class _Group:
    key: Tuple
    kv_heads: int
    head_dim: int
    window: Optional[int]
    pool: PagePool
    table: np.ndarray          # [max_slots, max_blocks] int32, -1 where no page


@dataclass
class _Request:
    slot: int
    length: int = 0
    # per group: number of leading blocks already given back (window) and blocks reserved so far
    released: List[int] = None
    reserved: List[int] = None


class CacheManager:
    @staticmethod
    def group_keys(needs: Sequence[Optional[CacheNeed]]) -> List[Tuple]:
        """The groups a list of needs forms, in the order the manager numbers them."""
        keys: List[Tuple] = []
        for need in needs:
            if need is not None and need.has_pages and need.group_key() not in keys:
                keys.append(need.group_key())
        return keys

    def __init__(self, needs: Sequence[Optional[CacheNeed]], cache_of: Sequence[Optional[int]], page_size: int,
                 num_pages, max_slots: int, max_context: int, device=None, kv_dtype=None):
        """needs[i]: CacheNeed of schedule entry i if it owns a cache, else None;
        cache_of[i]: the entry whose cache entry i reads, or None.
        ``num_pages``: the size of every group's pool, or one size per group (in the
        order of ``group_keys``). With ``device`` None no device memory is made
        (host-side tests)."""
        n_groups = len(self.group_keys(needs))
        if isinstance(num_pages, int):
            num_pages = [num_pages] * n_groups
        num_pages = [int(n) for n in num_pages]
        if len(num_pages) != n_groups:
            raise ValueError(f"{len(num_pages)} pool sizes were given for {n_groups} cache groups")
        self.page_size = page_size
        self.max_slots = max_slots
        self.max_blocks = -(-max_context // page_size)
        self.max_context = max_context
        self.device = device
        self.groups: List[_Group] = []
        self._entry_group: List[Optional[int]] = []
        key_to_group: Dict[Tuple, int] = {}
        for need in needs:
            if need is None or not need.has_pages:
                self._entry_group.append(None)
                continue
            key = need.group_key()
            if key not in key_to_group:
                key_to_group[key] = len(self.groups)
                self.groups.append(_Group(key, need.kv_heads, need.head_dim, need.window,
                                          PagePool(num_pages[len(self.groups)], len(self.groups)),
                                          np.full((max_slots, self.max_blocks), -1, dtype=np.int32)))
            self._entry_group.append(key_to_group[key])
        self._windowed = [gi for gi, g in enumerate(self.groups) if g.window is not None]   # groups that give pages back early
        self._free_slots: List[int] = list(range(max_slots - 1, -1, -1))
        self._requests: Dict[Hashable, _Request] = {}
        self._needs = list(needs)
        self._cache_of = list(cache_of)
        # device storage
        self._kv: List[Optional[Tuple[object, object]]] = [None] * len(needs)
        self._state: List[object] = [None] * len(needs)
        if device is not None:
            import torch

            for i, need in enumerate(needs):
                if need is None:
                    continue
                if need.has_pages:
                    shape = (num_pages[self._entry_group[i]], need.kv_heads, page_size, need.head_dim)
                    self._kv[i] = (torch.zeros(shape, dtype=kv_dtype, device=device),
                                   torch.zeros(shape, dtype=kv_dtype, device=device))
                if need.state_shape is not None:
                    self._state[i] = torch.zeros((max_slots,) + tuple(need.state_shape), dtype=torch.float32, device=device)

    # ---- sizes ----------------------------------------------------------
    @staticmethod
    def bytes_per_page(needs: Sequence[Optional[CacheNeed]], page_size: int, itemsize: int) -> List[int]:
        """Per group: device bytes one page id costs across the group's executions (K and V)."""
        keys = CacheManager.group_keys(needs)
        out = [0] * len(keys)
        for n in needs:
            if n is not None and n.has_pages:
                out[keys.index(n.group_key())] += 2 * page_size * n.kv_heads * n.head_dim * itemsize
        return out

    @staticmethod
    def most_pages_of_a_request(window: Optional[int], page_size: int, length: int, portion: int) -> int:
        """The most pages one request holds at a time in a group: all of its ``length`` tokens, or, behind a window,
        what a step of at most ``portion`` new tokens can still read (pages the window has passed were given back)."""
        full = -(-length // page_size)
        if window is None:
            return full
        return min(full, (window + max(portion, 1) - 2) // page_size + 2)

    def pool_pages(self) -> List[int]:
        return [g.pool.num_pages for g in self.groups]

    def free_pages(self) -> List[int]:
        return [g.pool.available for g in self.groups]

    def peak_pages(self, length: int, portion: int) -> List[int]:
        """Per group: the most pages a request that grows to ``length`` tokens, at most ``portion`` a step, holds at once."""
        return [self.most_pages_of_a_request(g.window, self.page_size, length, portion) for g in self.groups]

    def pages_held(self, rid: Hashable) -> List[int]:
        """Per group: pages the request holds now (what closing it gives back)."""
        r = self._requests.get(rid)
        if r is None:
            return [0] * len(self.groups)
        return [r.reserved[gi] - r.released[gi] for gi in range(len(self.groups))]

    def blocks_for(self, length: int) -> int:
        return -(-length // self.page_size)

    # ---- views ----------------------------------------------------------
    def views(self) -> List[Optional[CacheView]]:
        out: List[Optional[CacheView]] = []
        for i, need in enumerate(self._needs):
            src = self._cache_of[i]
            owner = i if src is None else src
            need_o = self._needs[owner]
            if need_o is None:
                out.append(None)
                continue
            kv = self._kv[owner] or (None, None)
            out.append(CacheView(group=self._entry_group[owner] if self._entry_group[owner] is not None else -1,
                                 k=kv[0], v=kv[1], page_size=self.page_size, writes=(src is None),
                                 state=self._state[owner], window=need_o.window))
        return out

    # ---- requests -------------------------------------------------------
    def is_open(self, rid: Hashable) -> bool:
        return rid in self._requests

    def length(self, rid: Hashable) -> int:
        return self._requests[rid].length

    def slot(self, rid: Hashable) -> int:
        return self._requests[rid].slot

    def lengths_and_slots(self, rids: Sequence[Hashable]) -> Tuple[List[int], List[int]]:
        """(tokens held, state slot) of each listed request, in one pass (a step asks this of every request it has)."""
        requests = self._requests
        found = [requests[rid] for rid in rids]
        return [r.length for r in found], [r.slot for r in found]

    @property
    def free_slots(self) -> int:
        return len(self._free_slots)

    @property
    def live(self) -> int:
        return len(self._requests)

    def open(self, rid: Hashable) -> int:
        if rid in self._requests:
            raise KeyError(f"request {rid!r} is already open")
        if not self._free_slots:
            raise NoFreeSlot(f"all {self.max_slots} slots are in use")
        slot = self._free_slots.pop()
        self._requests[rid] = _Request(slot, 0, [0] * len(self.groups), [0] * len(self.groups))
        for st in self._state:
            if st is not None:
                st[slot].zero_()
        return slot

    def _first_needed_block(self, g: _Group, length_before: int) -> int:
        """First block a query at position >= length_before can still read."""
        if g.window is None:
            return 0
        first_key = max(0, length_before - g.window + 1)
        return first_key // self.page_size

    def pages_wanted(self, rid: Hashable, new_len: int) -> List[int]:
        """Per group: pages that ``reserve`` would take for this request to reach new_len (a request that is not
        open counts as a new one)."""
        r = self._requests.get(rid)
        nb = self.blocks_for(new_len)
        if r is None:
            return [nb] * len(self.groups)
        return [max(0, nb - r.reserved[gi]) for gi in range(len(self.groups))]

    def free_after(self, batch: Sequence[Tuple[Hashable, int]], freed: Sequence[Hashable] = ()) -> List[int]:
        """Per group: pages that would be left (negative: missing) after ``reserve(batch)``, once the requests in
        ``freed`` were closed. Changes nothing."""
        n_groups = len(self.groups)
        free = [g.pool.available for g in self.groups]
        gone = set()
        for rid in freed:
            r = self._requests.get(rid)
            if r is not None and rid not in gone:
                gone.add(rid)
                for gi in range(n_groups):
                    free[gi] += r.reserved[gi] - r.released[gi]
        ps, requests = self.page_size, self._requests
        for rid, new_len in batch:
            nb = -(-new_len // ps)
            r = requests.get(rid)
            if r is None or rid in gone:
                for gi in range(n_groups):
                    free[gi] -= nb
            else:
                for gi in range(n_groups):
                    d = nb - r.reserved[gi]
                    if d > 0:
                        free[gi] -= d
        return free

    def fits(self, batch: Sequence[Tuple[Hashable, int]], freed: Sequence[Hashable] = (), at_most: Optional[int] = None) -> bool:
        """Would ``reserve(batch)`` succeed once the requests in ``freed`` were closed? Changes nothing.
        ``at_most``: an upper bound the caller knows for the pages any group can want (a request that grows by n
        tokens wants at most ceil(n / page_size)); if even that many are free, nothing is counted."""
        if at_most is not None and all(at_most <= g.pool.available for g in self.groups):
            return True
        return all(f >= 0 for f in self.free_after(batch, freed))

    def reserve(self, batch: Sequence[Tuple[Hashable, int]]) -> None:
        """Give every listed request pages up to its new length, or raise OutOfPages and change nothing."""
        n_groups = len(self.groups)
        want = [0] * n_groups
        grow = []                                   # (request, rid, blocks it must reach): only those that need pages
        ps, limit, requests = self.page_size, self.max_context, self._requests
        for rid, new_len in batch:
            r = requests[rid]
            if new_len > limit:
                raise ValueError(f"request {rid!r} would reach {new_len} tokens; the context limit is {limit}")
            if new_len < r.length:
                raise ValueError(f"request {rid!r} cannot shrink from {r.length} to {new_len}")
            nb = -(-new_len // ps)
            grows = False
            for gi in range(n_groups):
                d = nb - r.reserved[gi]
                if d > 0:
                    want[gi] += d
                    grows = True
            if grows:
                grow.append((r, rid, nb))
        for w, g in zip(want, self.groups):
            if w > g.pool.available:
                raise OutOfPages(w, g.pool.available, g.pool.group)
        for r, rid, nb in grow:
            for gi, g in enumerate(self.groups):
                n = nb - r.reserved[gi]
                if n > 0:
                    pages = g.pool.take(n, rid)
                    g.table[r.slot, r.reserved[gi]: r.reserved[gi] + n] = pages
                    r.reserved[gi] += n

    def commit(self, rid: Hashable, new_len: int) -> None:
        """The request now holds new_len tokens; pages a window has passed go back to the pool."""
        r = self._requests[rid]
        r.length = new_len
        for gi in self._windowed:
            g = self.groups[gi]
            first = min(self._first_needed_block(g, new_len), r.reserved[gi])
            if first > r.released[gi]:
                pages = [int(p) for p in g.table[r.slot, r.released[gi]: first]]
                g.pool.give_back(pages, rid)
                g.table[r.slot, r.released[gi]: first] = -1
                r.released[gi] = first

    def commit_many(self, batch: Sequence[Tuple[Hashable, int]]) -> None:
        """``commit`` for every (request, new length) of a step."""
        if self._windowed:
            for rid, new_len in batch:
                self.commit(rid, new_len)
            return
        requests = self._requests
        for rid, new_len in batch:
            requests[rid].length = new_len

    def close(self, rid: Hashable) -> None:
        r = self._requests.pop(rid)
        for gi, g in enumerate(self.groups):
            pages = [int(p) for p in g.table[r.slot, r.released[gi]: r.reserved[gi]]]
            g.pool.give_back(pages, rid)
            g.table[r.slot, :] = -1
        self._free_slots.append(r.slot)

    # ---- step inputs ----------------------------------------------------
    def table_rows(self, group: int, rids: Sequence[Hashable], width: Optional[int] = None,
                   slots: Optional[Sequence[int]] = None) -> np.ndarray:
        """[len(rids), width] int32 block-table rows (width: blocks of the longest listed request). ``slots``: the
        requests' slots, if the caller has them already."""
        g = self.groups[group]
        if slots is None:
            slots = [self._requests[rid].slot for rid in rids]
        if width is None:
            width = max([self._requests[rid].reserved[group] for rid in rids] + [1])
        return np.ascontiguousarray(g.table[slots, :width])

    # ---- checks (tests) -------------------------------------------------
    def check(self) -> None:
        for gi, g in enumerate(self.groups):
            g.pool.check()
            seen = {}
            for rid, r in self._requests.items():
                row = g.table[r.slot]
                live = [int(p) for p in row[r.released[gi]: r.reserved[gi]]]
                if any(p < 0 for p in live):
                    raise AssertionError(f"request {rid!r} has a hole in its live blocks")
                if any(int(p) >= 0 for p in row[: r.released[gi]]) or any(int(p) >= 0 for p in row[r.reserved[gi]:]):
                    raise AssertionError(f"request {rid!r} has table entries outside its live range")
                for p in live:
                    if p in seen:
                        raise AssertionError(f"page {p} is in the tables of {seen[p]!r} and {rid!r}")
                    seen[p] = rid
                    if g.pool.owner_of(p) != rid:
                        raise AssertionError(f"page {p} is in the table of {rid!r} but owned by {g.pool.owner_of(p)!r}")
            if len(seen) != g.pool.in_use:
                raise AssertionError(f"group {gi}: {g.pool.in_use} pages held, {len(seen)} in tables")
        slots = [r.slot for r in self._requests.values()]
        if len(set(slots)) != len(slots) or set(slots) & set(self._free_slots):
            raise AssertionError("a slot is held twice or both held and free")
        if len(slots) + len(self._free_slots) != self.max_slots:
            raise AssertionError("a slot was lost")
