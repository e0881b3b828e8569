"""The cache of a model: keys and values in pages, per-sequence state, and slots.

A *slot* stands for one live sequence.  A *lane* is the storage one run of a layer
uses (its keys and values for every sequence, its pooled keys, its state).  Lanes
with the same needs form a *group* that shares one storage tensor, one pool of
pages and one page table; lanes with other needs (another head count, a window
instead of all keys, pooled keys) form a group of their own.  A sequence's tokens
live in pages of 64 tokens; a key page is [kv_head][token_in_page][head_dim], a value
page is its transpose [kv_head][head_dim][token_in_page].  Pages and slots go back to the free lists when
a sequence ends and are used again as they are: only a slot's state is cleared, its
pages never are.  A group whose lanes look at a window of keys gives a sequence's pages
back as soon as every key in them has fallen out of the window of all later queries,
so what such a group holds per sequence is bounded by the window and the step size.

The reference keeps one sequence in one contiguous buffer per layer
(src/model/kvcache.cuh:7-26) and its per-sequence counters in host-side fields of each
layer object (src/model/minicpm4/minicpm4_kvcache.cuh:211-213).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch

from ..parts.base import PAGE_TOKENS, CacheNeeds
from .allocator import CacheFull, FreeList, HandleError

RELEASED = -1          # entry of a sequence's page list whose page went back to the pool


def pages_for(tokens: int) -> int:
    return (tokens + PAGE_TOKENS - 1) // PAGE_TOKENS


class CacheGroup:
    """Storage, pages and page table of the lanes that share one kind of needs."""

    def __init__(self, needs: CacheNeeds, lanes: List[int], n_pages: int, n_slots: int, max_pages_per_seq: int,
                 dtype: torch.dtype, device: torch.device, make=None):
        """``make(kind, shape, dtype, zero)`` gives the group its tensors (kind "state" or "pages"); by default they
        come from torch's allocator."""
        if make is None:
            def make(kind, shape, dt, zero):
                return (torch.zeros if zero else torch.empty)(shape, dtype=dt, device=device)
        self.needs = needs
        self.lanes = list(lanes)
        self.n_pages = n_pages
        self.max_pages_per_seq = max_pages_per_seq
        self.pages = FreeList(n_pages, "page")
        self.pages_of_slot: Dict[int, List[int]] = {}     # by logical page; RELEASED where the window has moved on
        self.first_live: Dict[int, int] = {}              # slot -> first logical page still held
        self.page_table = make("state", (n_slots, max_pages_per_seq), torch.int32, True)
        self._dirty: Dict[int, int] = {}      # slot -> first table column not yet on the device
        n = len(lanes)
        self.k = self.v = self.pooled = None
        if needs.kv_heads > 0:
            # zeros, not empty: a kernel may multiply a masked weight of 0 with whatever a page
            # holds beyond the sequence's end, and that has to be a finite number
            self.k = make("pages", (n, n_pages, needs.kv_heads, PAGE_TOKENS, needs.head_dim), dtype, True)
            self.v = make("pages", (n, n_pages, needs.kv_heads, needs.head_dim, PAGE_TOKENS), dtype, True)
            if needs.pooled_stride > 0:
                if PAGE_TOKENS % needs.pooled_stride:
                    raise ValueError(f"pooled-key stride {needs.pooled_stride} must divide the page size {PAGE_TOKENS}")
                per_page = PAGE_TOKENS // needs.pooled_stride
                # four bytes a dimension whatever the cache's type: fp32, or with a bf16 cache the two bf16 terms that the
                # selection's tensor-core scores take as operands (the kernels that write and read them know which)
                self.pooled = make("pages", (n, n_pages, needs.kv_heads, per_page, needs.head_dim), torch.float32, False)

    def bytes_per_token(self) -> int:
        if self.k is None:
            return 0
        per = 2 * self.needs.kv_heads * self.needs.head_dim * self.k.element_size() * len(self.lanes)
        if self.pooled is not None:
            per += self.needs.kv_heads * self.needs.head_dim * 4 * len(self.lanes) // self.needs.pooled_stride
        return per

    def reserve(self, slot: int, n_tokens: int) -> None:
        have = self.pages_of_slot.setdefault(slot, [])
        need = pages_for(n_tokens)
        if need > self.max_pages_per_seq:
            raise CacheFull(f"a sequence of {n_tokens} tokens needs {need} pages; the cache was sized for "
                            f"{self.max_pages_per_seq} pages ({self.max_pages_per_seq * PAGE_TOKENS} tokens) per sequence")
        if need > len(have):
            first_new = len(have)
            have.extend(self.pages.take(need - len(have)))
            self._dirty[slot] = min(self._dirty.get(slot, first_new), first_new)

    def release(self, slot: int) -> None:
        self.pages.give_back([p for p in self.pages_of_slot.pop(slot, []) if p != RELEASED])
        self.first_live.pop(slot, None)
        self._dirty.pop(slot, None)

    def pages_held(self, slot: int) -> int:
        return sum(1 for p in self.pages_of_slot.get(slot, []) if p != RELEASED)

    def trim(self, slot: int, length: int) -> int:
        """After a step that left the sequence ``length`` tokens long: gives back the pages all of whose keys
        lie before the window of every later query (a query at position p >= length sees the keys
        j > p - window).  The page table keeps the stale entries; no kernel follows them.  Returns the count."""
        window = self.needs.window
        if not window:
            return 0
        pages = self.pages_of_slot.get(slot)
        if not pages:
            return 0
        dead = min(max(0, length - window + 1) // PAGE_TOKENS, len(pages))
        first = self.first_live.get(slot, 0)
        if dead <= first:
            return 0
        self.pages.give_back(pages[first:dead])
        for i in range(first, dead):
            pages[i] = RELEASED
        self.first_live[slot] = dead
        return dead - first

    def sync(self) -> None:
        """Brings the device's page table up to date (pageable staging: no later host
        write can reach a copy that is still queued)."""
        for slot, first in self._dirty.items():
            pages = self.pages_of_slot[slot]
            first = max(first, self.first_live.get(slot, 0))
            if first >= len(pages):
                continue
            row = torch.tensor(pages[first:], dtype=torch.int32)
            self.page_table[slot, first:len(pages)].copy_(row)
        self._dirty.clear()


@dataclass
class Lane:
    """What one run of a layer sees of the cache."""

    index: int
    group: CacheGroup
    index_in_group: int
    state: Dict[str, torch.Tensor]

    @property
    def k(self) -> Optional[torch.Tensor]:
        return None if self.group.k is None else self.group.k[self.index_in_group]

    @property
    def v(self) -> Optional[torch.Tensor]:
        return None if self.group.v is None else self.group.v[self.index_in_group]

    @property
    def pooled(self) -> Optional[torch.Tensor]:
        return None if self.group.pooled is None else self.group.pooled[self.index_in_group]

    @property
    def page_table(self) -> torch.Tensor:
        return self.group.page_table


class Cache:
    def __init__(self, needs_per_lane: Sequence[CacheNeeds], max_tokens: int, dtype: torch.dtype,
                 device: "torch.device | str", n_slots: Optional[int] = None, max_seq_tokens: Optional[int] = None,
                 max_step_tokens: Optional[int] = None, state_region=None, page_region=None):
        """max_tokens: the most tokens live sequences hold together, each sequence's count
        rounded up to a whole page.  max_seq_tokens: the longest single sequence (default:
        all of max_tokens).  n_slots: the most live sequences (default: one per page, at
        most 1024).  max_step_tokens: the most tokens one step adds to a sequence; when given,
        a group with a window is sized for window + step tokens per slot instead of max_tokens.
        state_region / page_region: regions of an arena (cpmcu_b200.memory) that hold the page tables and the
        per-sequence state, and the pages; without them the tensors come from torch's allocator."""
        self.device = torch.device(device)
        make = None
        if state_region is not None or page_region is not None:
            def make(kind, shape, dt, zero):
                region = state_region if kind == "state" else page_region
                if region is None:
                    return (torch.zeros if zero else torch.empty)(shape, dtype=dt, device=self.device)
                return region.tensor(shape, dt, zero=zero, what="page tables and per-sequence state" if kind == "state"
                                     else "key-value pages")
        self.dtype = dtype
        n_pages = max(1, pages_for(max_tokens))
        self.n_pages = n_pages
        self.max_tokens = n_pages * PAGE_TOKENS
        self.n_slots = int(n_slots) if n_slots else min(n_pages, 1024)
        per_seq = pages_for(max_seq_tokens) if max_seq_tokens else n_pages
        self.max_pages_per_seq = max(1, min(per_seq, n_pages))
        self.slots = FreeList(self.n_slots, "slot")
        self.lengths: Dict[int, int] = {}

        self.groups: List[CacheGroup] = []
        by_key: Dict[tuple, List[int]] = {}
        for i, needs in enumerate(needs_per_lane):
            by_key.setdefault(needs.group_key(), []).append(i)
        self.lanes: List[Optional[Lane]] = [None] * len(needs_per_lane)
        for key, lane_ids in by_key.items():
            needs = needs_per_lane[lane_ids[0]]
            group_pages = n_pages
            if needs.window and max_step_tokens:
                # a sequence holds at most the pages its window and one step's tokens touch
                per_slot = pages_for(needs.window + int(max_step_tokens)) + 1
                group_pages = min(n_pages, self.n_slots * per_slot)
            group = CacheGroup(needs, lane_ids, group_pages, self.n_slots, self.max_pages_per_seq, dtype, self.device, make)
            self.groups.append(group)
            for j, lane_id in enumerate(lane_ids):
                state = {
                    name: (make("state", (self.n_slots, *shape), sdtype, True) if make is not None
                           else torch.zeros((self.n_slots, *shape), dtype=sdtype, device=self.device))
                    for name, (shape, sdtype) in needs_per_lane[lane_id].state.items()
                }
                self.lanes[lane_id] = Lane(lane_id, group, j, state)

    # ---- sequences ----
    def open_sequence(self) -> int:
        slot = self.slots.take(1)[0]
        self.lengths[slot] = 0
        for lane in self.lanes:
            for t in lane.state.values():
                t[slot].zero_()
        return slot

    def open_sequences(self, n: int) -> List[int]:
        if n > self.slots.n_free:
            raise CacheFull(f"{n} sequences wanted, {self.slots.n_free} of {self.n_slots} slots free")
        return [self.open_sequence() for _ in range(n)]

    def reserve(self, slot: int, new_length: int) -> None:
        """Makes room for the sequence to hold ``new_length`` tokens (all or nothing)."""
        if not self.slots.is_held(slot):
            raise HandleError(f"slot {slot} is not open")
        for g in self.groups:
            extra = pages_for(new_length) - len(g.pages_of_slot.get(slot, []))
            if extra > g.pages.n_free:
                raise CacheFull(f"growing a sequence to {new_length} tokens needs {extra} more pages, "
                                f"{g.pages.n_free} of {g.n_pages} are free (this group of layers holds "
                                f"{g.n_pages * PAGE_TOKENS} tokens)")
        for g in self.groups:
            g.reserve(slot, new_length)

    def check_room(self, growth: Sequence[tuple], step_tokens: int) -> None:
        """Raises CacheFull unless the sequences can all grow to their new lengths, (slot, new_length) each,
        when they do so in steps of at most ``step_tokens`` tokens with ``set_length`` after every step
        (which lets windowed groups give pages back on the way).  Takes nothing."""
        for g in self.groups:
            need = 0
            for slot, new_length in growth:
                if not self.slots.is_held(slot):
                    raise HandleError(f"slot {slot} is not open")
                extra = pages_for(new_length) - len(g.pages_of_slot.get(slot, []))
                if g.needs.window:
                    peak = pages_for(g.needs.window + int(step_tokens)) + 1      # most pages a sequence holds at once
                    extra = min(extra, peak - g.pages_held(slot))
                need += max(0, extra)
            if need > g.pages.n_free:
                raise CacheFull(f"the step needs {need} more pages, {g.pages.n_free} of {g.n_pages} are free "
                                f"(this group of layers holds {g.n_pages * PAGE_TOKENS} tokens)")

    def set_length(self, slot: int, length: int) -> None:
        """Called when a step is over and the sequence holds ``length`` tokens: windowed groups let go of the
        pages that no later query can see."""
        self.lengths[slot] = length
        for g in self.groups:
            g.trim(slot, length)

    def length(self, slot: int) -> int:
        return self.lengths[slot]

    def grow_by_one(self, slots: Sequence[int]) -> bool:
        """Room for one more token in each of ``slots`` (what a decode step needs): a page is taken only where the
        sequence's last page is full.  Returns True if a page table changed (``sync`` is then due).  All or nothing."""
        full = [s for s in slots if self.lengths[s] % PAGE_TOKENS == 0]
        if not full:
            return False
        for g in self.groups:
            need = sum(max(0, pages_for(self.lengths[s] + 1) - len(g.pages_of_slot.get(s, []))) for s in full)
            if need > g.pages.n_free:
                raise CacheFull(f"the step needs {need} more pages, {g.pages.n_free} of {g.n_pages} are free "
                                f"(this group of layers holds {g.n_pages * PAGE_TOKENS} tokens)")
        for s in full:
            self.reserve(s, self.lengths[s] + 1)
        return True

    def grown_by_one(self, slots: Sequence[int]) -> None:
        """The step is over: every sequence of ``slots`` holds one token more."""
        windowed = [g for g in self.groups if g.needs.window]
        for s in slots:
            n = self.lengths[s] + 1
            self.lengths[s] = n
            for g in windowed:
                g.trim(s, n)

    def close_sequence(self, slot: int) -> None:
        if not self.slots.is_held(slot):
            raise HandleError(f"slot {slot} is not open (closed twice?)")
        for g in self.groups:
            g.release(slot)
        del self.lengths[slot]
        self.slots.give_back([slot])

    def sync(self) -> None:
        for g in self.groups:
            g.sync()

    def lane(self, i: int) -> Lane:
        return self.lanes[i]

    # ---- accounting ----
    def tokens_held(self) -> int:
        return max((g.pages.n_held for g in self.groups), default=0) * PAGE_TOKENS

    def bytes_per_token(self) -> int:
        return sum(g.bytes_per_token() for g in self.groups)

    def check_consistent(self) -> None:
        """Every page is free or held by exactly one open sequence; raises otherwise."""
        for g in self.groups:
            seen = set()
            for slot, pages in g.pages_of_slot.items():
                if not self.slots.is_held(slot):
                    raise HandleError(f"pages held by closed slot {slot}")
                for p in pages:
                    if p == RELEASED:
                        continue
                    if p in seen:
                        raise HandleError(f"page {p} is held twice")
                    seen.add(p)
                    if not g.pages.is_held(p):
                        raise HandleError(f"page {p} is in use but marked free")
            if len(seen) != g.pages.n_held:
                raise HandleError(f"{g.pages.n_held - len(seen)} pages are lost (held by no sequence)")
