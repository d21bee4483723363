"""The cache of a model: paged keys and values per schedule entry, and fixed-size state per
sequence.

* A *sequence slot* stands for one live sequence: its length, its pages in every group and its
  row in the state area.  Slots are taken when a batch starts and given back when its
  sequences end; the lowest free slot and pages are taken first, so they are used again.
* Schedule entries whose mixers ask for the same keys and values (heads, head size, window)
  form a *group* with storage of its own: tensors ``k, v [entry, page, kv head, PAGE, head_dim]``,
  one free list of pages and one page table per sequence, shared by the group's entries.
  A page holds PAGE = 64 consecutive positions of one sequence.
* A group with a window gives a page back as soon as all its positions lie before every
  window that a later token can have, so in steady state it holds about ``window`` positions
  per sequence.
* State: ``state [entry with state, slot, elems]`` (float32 unless the mixer asks otherwise), zeroed when a slot is taken.
* Values may have another head size and another number of heads than keys (``KVNeed.v_head_dim``, ``v_heads``): the
  pools are then shaped accordingly (this library's attention kernels take equal shapes; a mixer that asks for
  others brings the kernel that reads them).
* Beside what sequences hold there is one *idle* slot with one page in every group (``idle_slot``,
  ``idle_page``: the index after the last real one): a step that is padded to a fixed number of rows
  (a captured decode step of a bucket of rows) lets its idle rows read and write there, so that
  kernels need no notion of a row that is not there.  It takes no page and no slot from the sequences.

pico-engine allocates a fresh zeroed (kv head, capacity, head_dim) pair per layer for every
request (src/pico_engine/engine.py:119-121, 316) and keeps its recurrent model's per-layer
state in fixed tensors (engine.py:101-109); neither is reused across requests there.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from .needs import CacheNeeds, KVNeed
from .pages import CacheFull, CacheStateError, FreeList

PAGE = 64


def pages_for(tokens: int) -> int:
    return (tokens + PAGE - 1) // PAGE


@dataclass
class KVGroup:
    need: KVNeed
    entries: List[int]                    # schedule entries that own storage here, in order
    k: Optional[torch.Tensor]             # [len(entries), pages, n_kv_heads, PAGE, head_dim]
    v: Optional[torch.Tensor]
    pages: FreeList
    table: Dict[int, List[int]]           # slot -> physical page of each logical page (-1: given back)

    def bytes(self) -> int:
        return 0 if self.k is None else (self.k.numel() + self.v.numel()) * self.k.element_size()      # with the idle page


class Cache:
    """``needs[e]`` is what schedule entry ``e`` asks for (None for an entry that reads
    another entry's cache or needs nothing).  ``max_tokens`` is the most tokens live sequences
    hold at any time, each sequence's count rounded up to PAGE."""

    def __init__(self, needs: Sequence[Optional[CacheNeeds]], max_tokens: int, max_seqs: int, dtype: torch.dtype,
                 device, allocate: bool = True):
        if max_tokens <= 0 or max_seqs <= 0:
            raise ValueError("the cache needs room for at least one token and one sequence")
        self.dtype, self.device = dtype, torch.device(device)
        self.n_pages = pages_for(max_tokens)
        self.max_seqs = max_seqs
        self.slots = FreeList(max_seqs, "sequence slot")
        self.lengths: Dict[int, int] = {}
        self.groups: List[KVGroup] = []
        self.group_of: Dict[int, int] = {}        # schedule entry -> group
        self.index_in_group: Dict[int, int] = {}
        by_need: Dict[KVNeed, int] = {}
        for e, n in enumerate(needs):
            if n is None or n.kv is None:
                continue
            if n.kv not in by_need:
                by_need[n.kv] = len(self.groups)
                self.groups.append(KVGroup(n.kv, [], None, None, FreeList(self.n_pages, "page"), {}))
            g = by_need[n.kv]
            self.group_of[e] = g
            self.index_in_group[e] = len(self.groups[g].entries)
            self.groups[g].entries.append(e)
        self.state_entries = [e for e, n in enumerate(needs) if n is not None and n.state_elems > 0]
        self.state: Dict[int, torch.Tensor] = {}
        self.idle_slot, self.idle_page = max_seqs, self.n_pages       # one past the slots and pages that sequences use
        if allocate:
            for g in self.groups:
                v_heads, v_dim = g.need.value_shape
                g.k = torch.zeros((len(g.entries), self.n_pages + 1, g.need.n_kv_heads, PAGE, g.need.head_dim),
                                  dtype=dtype, device=self.device)
                g.v = torch.zeros((len(g.entries), self.n_pages + 1, v_heads, PAGE, v_dim), dtype=dtype, device=self.device)
            for e in self.state_entries:
                kind = needs[e].state_dtype
                if kind not in ("float32", "bfloat16", "engine"):
                    raise ValueError(f"schedule entry {e}: state_dtype must be float32, bfloat16 or engine, not {kind!r}")
                sd = dtype if kind == "engine" else getattr(torch, kind)
                self.state[e] = torch.zeros(max_seqs + 1, needs[e].state_elems, dtype=sd, device=self.device)

    # ------------------------------------------------------------------ sequences
    def open(self) -> int:
        """A slot for a new, empty sequence."""
        (slot,) = self.slots.take(1)
        self.lengths[slot] = 0
        for g in self.groups:
            g.table[slot] = []
        for t in self.state.values():
            t[slot].zero_()
        return slot

    def close(self, slot: int) -> None:
        """Give back the slot and everything it holds."""
        if slot not in self.lengths:
            raise CacheStateError(f"sequence slot {slot} is closed but is not open")
        for g in self.groups:
            g.pages.give(p for p in g.table.pop(slot) if p >= 0)
        del self.lengths[slot]
        self.slots.give([slot])

    def length(self, slot: int) -> int:
        return 0 if slot == self.idle_slot else self.lengths[slot]

    def snapshot_state(self) -> Dict[int, torch.Tensor]:
        """A copy of the per-sequence state of every entry that has some (for running a step on trial)."""
        return {e: t.clone() for e, t in self.state.items()}

    def restore_state(self, snapshot: Dict[int, torch.Tensor]) -> None:
        for e, t in snapshot.items():
            self.state[e].copy_(t)

    def held_tokens(self) -> int:
        """Tokens held by live sequences, each rounded up to PAGE."""
        return sum(pages_for(n) * PAGE for n in self.lengths.values())

    # ------------------------------------------------------------------ one step
    def reserve(self, slot: int, n_new: int) -> None:
        """Pages for positions ``length .. length + n_new - 1`` of the sequence, in every group."""
        want = pages_for(self.lengths[slot] + n_new)
        for g in self.groups:
            have = len(g.table[slot])
            if want > have:
                g.table[slot].extend(g.pages.take(want - have))

    def advance(self, slot: int, n_new: int) -> None:
        """The step has written ``n_new`` more positions.  Windowed groups give back the pages
        that no later token can see: a token at position p >= length sees keys >= p - window + 1."""
        self.lengths[slot] += n_new
        first_needed = self.lengths[slot]          # the next query's position
        for g in self.groups:
            if g.need.window is None:
                continue
            oldest = first_needed - g.need.window + 1
            row = g.table[slot]
            for pi in range(len(row)):
                if (pi + 1) * PAGE - 1 >= oldest:
                    break
                if row[pi] >= 0:
                    g.pages.give([row[pi]])
                    row[pi] = -1

    def page_table(self, group: int, slots: Sequence[int], width: Optional[int] = None) -> np.ndarray:
        """int32 [len(slots), width]: physical page of each logical page, -1 where there is none."""
        g = self.groups[group]
        width = width or max(1, max(len(g.table[s]) for s in slots if s != self.idle_slot) if any(s != self.idle_slot for s in slots) else 1)
        out = np.full((len(slots), width), -1, dtype=np.int32)
        for r, s in enumerate(slots):
            if s == self.idle_slot:
                out[r, 0] = self.idle_page
                continue
            row = g.table[s]
            if len(row) > width:
                raise CacheFull(f"sequence slot {s} holds {len(row)} pages, the table has room for {width}")
            out[r, :len(row)] = row
        return out

    # ------------------------------------------------------------------ what a mixer sees
    def pools(self, entry: int):
        """(k, v) [page, kv head, PAGE, head_dim] of a schedule entry that owns storage."""
        g = self.groups[self.group_of[entry]]
        i = self.index_in_group[entry]
        return g.k[i], g.v[i]

    def state_of(self, entry: int) -> Optional[torch.Tensor]:
        """[slot, elems] float32 of an entry with state, else None."""
        return self.state.get(entry)

    def bytes(self) -> int:
        return sum(g.bytes() for g in self.groups) + sum(t.numel() * t.element_size() for t in self.state.values())

    def check(self) -> None:
        """Invariants of the bookkeeping: nothing lost, nothing held twice."""
        self.slots.check()
        if sorted(self.lengths) != sorted(i for i in range(self.max_seqs) if self.slots._held[i]):
            raise CacheStateError("open sequences and held slots differ")
        for g in self.groups:
            g.pages.check()
            held = [p for row in g.table.values() for p in row if p >= 0]
            if len(held) != len(set(held)):
                raise CacheStateError("a page belongs to two sequences")
            if len(held) != g.pages.held_count:
                raise CacheStateError("pages are held that no sequence owns")
