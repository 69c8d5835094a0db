"""The cache of a model: a slot for each live sequence with its own length,
keys and values for each place of the schedule that writes some, and a
fixed-size state area per slot for mixers that keep state.

Places with the same needs (KVSpec) form a group; a group owns its page pool,
its storage and, per slot, its list of pages.  A group with a window gives back
pages whose keys every later query has left behind.  Slots and pages are reused
by later sequences without being cleared: every read is bounded by the
sequence's length.  State areas are zeroed when a slot is taken.

The reference keeps one dense buffer [batch][layer][max_seq][kv_head][head_dim]
with one position counter for all rows
(crates/janus-engine/src/compute/cache/core.rs:15,47,212-230) and errors when a
position passes the end (core.rs:283-288); here the error is `CacheFull`,
raised before anything is launched.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..parts.base import CacheSpec, KVSpec, StateSpec
from .pages import PAGE_SIZE, CacheFull, PagePool


class KVGroup:
    """Storage of all places that share one KVSpec: per place K and V of shape
    [n_pages, n_kv_heads, PAGE_SIZE, head_dim]."""

    def __init__(self, spec: KVSpec, places: Sequence[int], n_pages: int, n_slots: int,
                 dtype: torch.dtype, device: torch.device):
        self.spec, self.places = spec, list(places)
        self.pool = PagePool(n_pages)
        self.page_size = PAGE_SIZE
        shape = (n_pages, spec.n_kv_heads, PAGE_SIZE, spec.head_dim)
        self.k: Dict[int, torch.Tensor] = {p: torch.zeros(shape, dtype=dtype, device=device) for p in self.places}
        self.v: Dict[int, torch.Tensor] = {p: torch.zeros(shape, dtype=dtype, device=device) for p in self.places}
        # pages[slot][i] holds keys [i*PAGE, (i+1)*PAGE); -1 once a window has passed it
        self.pages: List[List[int]] = [[] for _ in range(n_slots)]

    def reserve(self, slot: int, new_length: int) -> None:
        need = (new_length + PAGE_SIZE - 1) // PAGE_SIZE
        pages = self.pages[slot]
        if need - len(pages) > self.pool.n_free:
            raise CacheFull(
                f"the cache has {self.pool.n_free} free pages of {PAGE_SIZE} tokens, "
                f"{need - len(pages)} more are needed to hold {new_length} tokens in slot {slot}")
        while len(pages) < need:
            pages.append(self.pool.take())

    def release_passed(self, slot: int, length: int) -> None:
        """With a window w, the next query (position `length`) reads keys
        > length - w; pages wholly at or below that are given back."""
        w = self.spec.window
        if w <= 0:
            return
        pages = self.pages[slot]
        first_needed = max(0, length - w + 1)
        for i in range(min(len(pages), first_needed // PAGE_SIZE)):
            if pages[i] >= 0:
                self.pool.give_back(pages[i])
                pages[i] = -1

    def release_all(self, slot: int) -> None:
        for p in self.pages[slot]:
            if p >= 0:
                self.pool.give_back(p)
        self.pages[slot] = []

    def dest_rows(self, slot: int, start: int, n: int) -> np.ndarray:
        pos = np.arange(start, start + n, dtype=np.int64)
        pages = np.asarray(self.pages[slot], dtype=np.int64)
        return (pages[pos // PAGE_SIZE] * PAGE_SIZE + pos % PAGE_SIZE).astype(np.int32)


@dataclass
class GroupStepView:
    """What a step hands a mixer about its group: where each new token's keys go
    and, per sequence of the step, the pages of its keys."""
    dest_rows: torch.Tensor        # int32 [T]
    block_table: torch.Tensor      # int32 [n_seqs, max_pages]
    page_size: int


@dataclass
class CacheView:
    """One place's view during a step."""
    k: Optional[torch.Tensor] = None
    v: Optional[torch.Tensor] = None
    group: Optional[GroupStepView] = None
    state: Optional[torch.Tensor] = None      # float32 [n_slots, *shape]


class SequenceCache:
    def __init__(self, place_specs: Sequence[CacheSpec], max_tokens: int, n_slots: int,
                 dtype: torch.dtype, device: torch.device):
        """place_specs[i] is what the i-th place of the schedule needs (None if
        it reads another place's cache or needs nothing).  `max_tokens` is the
        most tokens the live sequences hold at any time, each sequence's count
        rounded up to a multiple of PAGE_SIZE."""
        self.n_slots = int(n_slots)
        self.dtype, self.device = dtype, device
        n_pages = max(1, (int(max_tokens) + PAGE_SIZE - 1) // PAGE_SIZE)
        self.n_pages = n_pages
        by_spec: Dict[KVSpec, List[int]] = {}
        self.states: Dict[int, torch.Tensor] = {}
        for place, spec in enumerate(place_specs):
            if isinstance(spec, KVSpec):
                by_spec.setdefault(spec, []).append(place)
            elif isinstance(spec, StateSpec):
                self.states[place] = torch.zeros((self.n_slots, *spec.shape), dtype=torch.float32, device=device)
            elif spec is not None:
                raise TypeError(f"place {place}: unknown cache spec {spec!r}")
        self.groups: List[KVGroup] = [KVGroup(spec, places, n_pages, self.n_slots, dtype, device)
                                      for spec, places in by_spec.items()]
        self.group_of_place: Dict[int, int] = {p: gi for gi, g in enumerate(self.groups) for p in g.places}
        self._free_slots: List[int] = list(range(self.n_slots - 1, -1, -1))
        self._live = [False] * self.n_slots
        self.lengths = [0] * self.n_slots
        self.epochs = [0] * self.n_slots      # bumped each time a slot is taken: tells occupants apart

    # -- slots ---------------------------------------------------------------
    @property
    def n_free_slots(self) -> int:
        return len(self._free_slots)

    def alloc_slot(self) -> int:
        if not self._free_slots:
            raise CacheFull(f"all {self.n_slots} sequence slots are in use")
        slot = self._free_slots.pop()
        self._live[slot] = True
        self.lengths[slot] = 0
        self.epochs[slot] += 1
        for st in self.states.values():
            st[slot].zero_()
        return slot

    def free_slot(self, slot: int) -> None:
        self._require_live(slot)
        for g in self.groups:
            g.release_all(slot)
        self._live[slot] = False
        self.lengths[slot] = 0
        self._free_slots.append(slot)

    def is_live(self, slot: int) -> bool:
        return 0 <= slot < self.n_slots and self._live[slot]

    def _require_live(self, slot: int) -> None:
        if not self.is_live(slot):
            raise ValueError(f"slot {slot} is not held by a live sequence")

    def length(self, slot: int) -> int:
        self._require_live(slot)
        return self.lengths[slot]

    # -- growth --------------------------------------------------------------
    def reserve(self, slot: int, n_new: int) -> None:
        """Make room for n_new more tokens in every group, or raise CacheFull
        and leave the slot as it was."""
        self._require_live(slot)
        new_length = self.lengths[slot] + n_new
        before = [len(g.pages[slot]) for g in self.groups]
        try:
            for g in self.groups:
                g.reserve(slot, new_length)
        except CacheFull:
            for g, n in zip(self.groups, before):
                while len(g.pages[slot]) > n:
                    g.pool.give_back(g.pages[slot].pop())
            raise

    def advance(self, slot: int, n_new: int) -> None:
        self._require_live(slot)
        self.lengths[slot] += n_new
        for g in self.groups:
            g.release_passed(slot, self.lengths[slot])

    def check(self) -> None:
        """Consistency of slots and pages (used by tests)."""
        if len(set(self._free_slots)) != len(self._free_slots):
            raise AssertionError("a slot is in the free list twice")
        for s in range(self.n_slots):
            if self._live[s] == (s in self._free_slots):
                raise AssertionError(f"slot {s} is {'live and free' if self._live[s] else 'lost'}")
        for g in self.groups:
            g.pool.check()
            held = [p for s in range(self.n_slots) for p in g.pages[s] if p >= 0]
            if len(held) != len(set(held)):
                raise AssertionError("a page is held by two sequences")
            if len(held) != g.pool.n_held:
                raise AssertionError(f"{g.pool.n_held} pages are held but sequences list {len(held)}")
            for s in range(self.n_slots):
                if not self._live[s] and g.pages[s]:
                    raise AssertionError(f"free slot {s} still lists pages")
