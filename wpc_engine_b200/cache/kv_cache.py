"""The cache: a slot for each live sequence, keys and values for each cache layer in pages,
and per-sequence records of fixed size.

Storage is grouped by what the layers need (`KVSpec` with or without a window, `StateSpec`):
every group has tensors and a page pool of its own.  A sequence holds, in each key/value
group, the pages that cover its positions; in a group with a window the pages that lie wholly
before the window are given back after every step.  Position p of a sequence lives in page
`table[p // PAGE]` at row `p % PAGE`.

The reference keeps one growable vector per layer and KV head for its single sequence
(wpc-runtime/src/model.rs:38-62); slots, pages and groups have no counterpart there.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch

from ..constants import PAGE          # positions per page; `--max-tokens` is counted in these units
from ..parts.base import KVSpec, StateSpec
from .pages import CacheError, FreeList


def pages_for(n_tokens: int) -> int:
    return (n_tokens + PAGE - 1) // PAGE


@dataclass
class KVView:
    """What a mixer sees of the cache in one step, for one cache layer."""
    k_pages: torch.Tensor        # [n_pages, n_kv_heads, PAGE, head_dim]
    v_pages: torch.Tensor        # [n_pages, n_kv_heads, PAGE, value_dim]
    page_table: torch.Tensor     # int32 [B, width]: page of block i of sequence b, -1 if none
    writes: bool = True


@dataclass
class StateView:
    """The fixed-size records of one cache layer; row `slots[b]` belongs to sequence b."""
    state: torch.Tensor          # [n_slots, *shape]
    slots: torch.Tensor          # int32 [B]
    writes: bool = True


def window_pages(window: int, max_step_tokens: int) -> int:
    """The most pages that one sequence holds in a group with `window` when no step brings it
    more than max_step_tokens tokens: the blocks from the first position that the step's first
    query sees to the step's last position."""
    return pages_for(window + max_step_tokens - 1) + 1


class KVGroup:
    """The keys and values of the cache layers that share one `KVSpec`: tensors and a page pool of
    the group's own.  `pages_per_sequence` (windowed groups of an engine whose steps are bounded)
    is the most pages that one sequence ever holds here, None where its length alone bounds it."""

    def __init__(self, spec: KVSpec, n_layers: int, n_pages: int, dtype: torch.dtype, device,
                 pages_per_sequence: Optional[int] = None):
        self.spec = spec
        self.n_layers = n_layers
        self.n_pages = n_pages
        self.pages_per_sequence = pages_per_sequence
        self.k = torch.zeros((n_layers, n_pages, spec.n_kv_heads, PAGE, spec.head_dim), dtype=dtype, device=device)
        self.v = torch.zeros((n_layers, n_pages, spec.n_kv_heads, PAGE, spec.value_dim), dtype=dtype, device=device)
        self.pool = FreeList(n_pages, "page")
        self.tables: Dict[int, List[int]] = {}        # slot -> page of each block (-1: given back)

    def pages_needed(self, n_tokens: int) -> int:
        """Pages that a sequence grown to n_tokens positions holds here at most."""
        need = pages_for(n_tokens)
        return need if self.pages_per_sequence is None else min(need, self.pages_per_sequence)

    def open(self, slot: int) -> None:
        self.tables[slot] = []

    def reserve(self, slot: int, new_len: int) -> None:
        table = self.tables[slot]
        need = pages_for(new_len) - len(table)
        if need > 0:
            table.extend(self.pool.take_many(need))

    def release_beyond(self, slot: int, length: int) -> None:
        """Gives back the pages behind the last position of a sequence of `length` positions
        (what `reserve` took for a step that did not run)."""
        table = self.tables[slot]
        while len(table) > pages_for(length):
            page = table.pop()
            if page >= 0:
                self.pool.give_back(page)

    def trim(self, slot: int, length: int) -> None:
        """Gives back the pages that no later query of a windowed group can see."""
        if self.spec.window is None:
            return
        first_visible = max(0, length - self.spec.window + 1)   # of the next query, at `length`
        table = self.tables[slot]
        for block in range(first_visible // PAGE):
            if table[block] >= 0:
                self.pool.give_back(table[block])
                table[block] = -1

    def close(self, slot: int) -> None:
        for page in self.tables.pop(slot):
            if page >= 0:
                self.pool.give_back(page)


class StateGroup:
    def __init__(self, spec: StateSpec, n_layers: int, n_slots: int, device):
        self.spec = spec
        self.n_layers = n_layers
        dtype = getattr(torch, spec.dtype)
        self.state = torch.zeros((n_layers, n_slots) + tuple(spec.shape), dtype=dtype, device=device)

    def open(self, slot: int) -> None:
        self.state[:, slot].zero_()


class SequenceCache:
    """Slots, groups and lengths.  `cache_specs[i]` is what cache layer i keeps (None: nothing).

    max_tokens: the most positions that live sequences hold at any time, each sequence rounded
    up to whole pages.  It sizes the pool of every key/value group that keeps all positions.
    A group with a window needs less when no step brings a sequence more than `max_step_tokens`
    tokens (None: unbounded): then each of the `max_sequences` slots holds at most
    `window_pages(window, max_step_tokens)` pages there, and the pool is that small.  A model
    without key/value groups has no pages at all.
    """

    def __init__(self, cache_specs: Sequence[object], max_tokens: int, dtype: torch.dtype, device,
                 max_sequences: Optional[int] = None, max_step_tokens: Optional[int] = None):
        self.device = device
        self.n_pages = pages_for(max_tokens)
        if self.n_pages < 1:
            raise CacheError(f"max_tokens {max_tokens} gives no page")
        self.n_slots = int(max_sequences) if max_sequences else self.n_pages
        self.max_step_tokens = None if max_step_tokens is None else int(max_step_tokens)
        self.slots = FreeList(self.n_slots, "slot")
        self.lengths: Dict[int, int] = {}
        self.groups: List[object] = []
        self.layer_group: List[Optional[int]] = []       # cache layer -> group
        self.layer_index: List[Optional[int]] = []       # cache layer -> layer within the group
        by_spec: Dict[object, List[int]] = {}
        for i, spec in enumerate(cache_specs):
            if spec is not None:
                by_spec.setdefault(spec, []).append(i)
        self.layer_group = [None] * len(cache_specs)
        self.layer_index = [None] * len(cache_specs)
        for spec, layers in by_spec.items():
            if isinstance(spec, KVSpec):
                per_seq, n_pages = None, self.n_pages
                if spec.window is not None and self.max_step_tokens is not None:
                    per_seq = window_pages(spec.window, self.max_step_tokens)
                    n_pages = min(self.n_pages, self.n_slots * per_seq)
                group = KVGroup(spec, len(layers), n_pages, dtype, device, per_seq)
            elif isinstance(spec, StateSpec):
                group = StateGroup(spec, len(layers), self.n_slots, device)
            else:
                raise CacheError(f"unknown cache spec {spec!r}")
            g = len(self.groups)
            self.groups.append(group)
            for j, layer in enumerate(layers):
                self.layer_group[layer] = g
                self.layer_index[layer] = j
        # position, sampler key, sampler counter, tokens generated: one int64 row per slot
        self.seq_state = torch.zeros((self.n_slots, 4), dtype=torch.int64, device=device)

    # -- slots -----------------------------------------------------------------------------
    def open(self) -> int:
        slot = self.slots.take()
        self.lengths[slot] = 0
        for g in self.groups:
            g.open(slot)
        return slot

    def close(self, slot: int) -> None:
        if slot not in self.lengths:
            raise CacheError(f"slot {slot} is closed but is not open")
        for g in self.groups:
            if isinstance(g, KVGroup):
                g.close(slot)
        del self.lengths[slot]
        self.slots.give_back(slot)

    def length(self, slot: int) -> int:
        return self.lengths[slot]

    # -- a step ------------------------------------------------------------------------------
    def reserve(self, slot: int, n_new: int) -> int:
        """Makes room for n_new more positions; returns the position of the first of them."""
        start = self.lengths[slot]
        for g in self.groups:
            if isinstance(g, KVGroup):
                g.reserve(slot, start + n_new)
        return start

    def release_unused(self, slot: int) -> None:
        """Undoes `reserve` for a step that did not run: pages behind the sequence's length go back."""
        for g in self.groups:
            if isinstance(g, KVGroup):
                g.release_beyond(slot, self.lengths[slot])

    def fits(self, token_counts: Sequence[int]) -> bool:
        """Whether sequences grown to these many positions can all live in the cache at once."""
        if len(token_counts) > self.n_slots:
            return False
        for g in self.groups:
            if isinstance(g, KVGroup) and sum(g.pages_needed(n) for n in token_counts) > g.n_pages:
                return False
        return True

    def commit(self, slot: int, n_new: int) -> None:
        self.lengths[slot] += n_new
        for g in self.groups:
            if isinstance(g, KVGroup):
                g.trim(slot, self.lengths[slot])

    def table_width(self, slots: Sequence[int]) -> int:
        width = 1
        for g in self.groups:
            if isinstance(g, KVGroup):
                for s in slots:
                    width = max(width, len(g.tables[s]))
        return width

    def page_table_rows(self, group: int, slots: Sequence[int], width: int) -> List[List[int]]:
        g = self.groups[group]
        return [g.tables[s] + [-1] * (width - len(g.tables[s])) for s in slots]

    def kv_groups(self) -> List[int]:
        return [i for i, g in enumerate(self.groups) if isinstance(g, KVGroup)]

    def check(self) -> None:
        """No slot or page lost, held twice or free twice; held pages belong to open slots."""
        self.slots.check()
        for g in self.groups:
            if not isinstance(g, KVGroup):
                continue
            g.pool.check()
            owned = [p for t in g.tables.values() for p in t if p >= 0]
            if len(owned) != len(set(owned)):
                raise CacheError("a page belongs to two sequences")
            if len(owned) != g.pool.n_held:
                raise CacheError(f"{g.pool.n_held} pages are held but sequences own {len(owned)}")
            if set(g.tables) != set(self.lengths):
                raise CacheError("page tables and open slots differ")
