"""What one step runs: the packed tokens of a batch and where they live in the cache.

`plan_step` turns the host's view (per sequence: slot, new tokens, wanted places) into one
block of int32 metadata, laid out so that a single host-to-device copy moves it, and
`StepContext` is the device's view of that block that every part receives.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch


@dataclass
class SequenceStep:
    """One sequence's share of a step."""
    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = ()        # places among `tokens` whose logits are asked for


@dataclass
class StepLayout:
    """Offsets (in int32 elements) of each field inside the metadata block."""
    n_tokens: int
    n_seqs: int
    n_want: int
    table_width: int
    n_kv_groups: int
    tokens: int = 0
    positions: int = 0
    seq_of_token: int = 0
    cu_seqlens: int = 0
    ctx_lens: int = 0
    slots: int = 0
    want_rows: int = 0
    tables: int = 0
    total: int = 0

    def __post_init__(self):
        def align(x):       # 16-byte alignment of every field
            return (x + 3) // 4 * 4
        off = 0
        self.tokens = off; off = align(off + self.n_tokens)
        self.positions = off; off = align(off + self.n_tokens)
        self.seq_of_token = off; off = align(off + self.n_tokens)
        self.cu_seqlens = off; off = align(off + self.n_seqs + 1)
        self.ctx_lens = off; off = align(off + self.n_seqs)
        self.slots = off; off = align(off + self.n_seqs)
        self.want_rows = off; off = align(off + max(self.n_want, 1))
        self.tables = off; off = align(off + self.n_kv_groups * self.n_seqs * self.table_width)
        self.total = off


@dataclass
class StepPlan:
    layout: StepLayout
    host: np.ndarray                  # int32 [layout.total]
    max_new_tokens: int
    max_ctx_len: int
    is_decode: bool
    starts: List[int]                 # position of each sequence's first new token


def plan_step(entries: Sequence[SequenceStep], starts: Sequence[int],
              table_rows: Sequence[Sequence[Sequence[int]]], table_width: int,
              out: Optional[np.ndarray] = None) -> StepPlan:
    """starts[b]: the length of sequence b before this step.  table_rows[g][b]: the page table
    row (already `table_width` wide) of sequence b in key/value group g."""
    n_seqs = len(entries)
    if n_seqs == 0:
        raise ValueError("a step needs at least one sequence")
    lens = [len(e.tokens) for e in entries]
    if min(lens) < 1:
        raise ValueError("every sequence of a step brings at least one token")
    n_tokens = sum(lens)
    n_want = sum(len(e.want) for e in entries)
    lay = StepLayout(n_tokens, n_seqs, n_want, table_width, len(table_rows))
    host = out[: lay.total] if out is not None else np.empty(lay.total, dtype=np.int32)
    host[:] = 0
    t = 0
    w = 0
    for b, e in enumerate(entries):
        n = lens[b]
        host[lay.tokens + t: lay.tokens + t + n] = np.asarray(e.tokens, dtype=np.int64)
        host[lay.positions + t: lay.positions + t + n] = np.arange(starts[b], starts[b] + n)
        host[lay.seq_of_token + t: lay.seq_of_token + t + n] = b
        host[lay.cu_seqlens + b] = t
        host[lay.ctx_lens + b] = starts[b] + n
        host[lay.slots + b] = e.slot
        for place in e.want:
            if not 0 <= place < n:
                raise ValueError(f"wanted place {place} is outside the {n} tokens of this step")
            host[lay.want_rows + w] = t + place
            w += 1
        t += n
    host[lay.cu_seqlens + n_seqs] = t
    for g, rows in enumerate(table_rows):
        base = lay.tables + g * n_seqs * table_width
        host[base: base + n_seqs * table_width] = np.asarray(rows, dtype=np.int32).reshape(-1)
    return StepPlan(lay, host, max(lens), max(s + n for s, n in zip(starts, lens)),
                    all(n == 1 for n in lens), list(starts))


@dataclass
class StepContext:
    """The device's view of a step; parts read what they need from it."""
    act_dtype: torch.dtype
    n_tokens: int
    n_seqs: int
    tokens: torch.Tensor            # int32 [T]
    positions: torch.Tensor         # int32 [T] absolute position of each token
    seq_of_token: torch.Tensor      # int32 [T] which sequence of the step a token belongs to
    cu_seqlens: torch.Tensor        # int32 [B + 1] first token of each sequence
    ctx_lens: torch.Tensor          # int32 [B] length of each sequence after this step
    slots: torch.Tensor             # int32 [B]
    want_rows: torch.Tensor         # int32 [n_want] token rows whose logits are wanted
    page_tables: List[torch.Tensor]  # per key/value group: int32 [B, table_width]
    max_new_tokens: int
    max_ctx_len: int
    is_decode: bool
    new_tokens_host: Optional[List[int]] = None   # tokens that each sequence brings, on the host (all 1 in a graph)
    shared: Dict[object, object] = field(default_factory=dict)   # per-step tables of the parts


def context_from(meta: torch.Tensor, lay: StepLayout, act_dtype: torch.dtype, max_new_tokens: int,
                 max_ctx_len: int, is_decode: bool, new_tokens_host: Optional[List[int]] = None) -> StepContext:
    def view(off, n):
        return meta[off: off + n]
    tables = []
    for g in range(lay.n_kv_groups):
        base = lay.tables + g * lay.n_seqs * lay.table_width
        tables.append(view(base, lay.n_seqs * lay.table_width).view(lay.n_seqs, lay.table_width))
    return StepContext(
        act_dtype=act_dtype, n_tokens=lay.n_tokens, n_seqs=lay.n_seqs,
        tokens=view(lay.tokens, lay.n_tokens), positions=view(lay.positions, lay.n_tokens),
        seq_of_token=view(lay.seq_of_token, lay.n_tokens),
        cu_seqlens=view(lay.cu_seqlens, lay.n_seqs + 1), ctx_lens=view(lay.ctx_lens, lay.n_seqs),
        slots=view(lay.slots, lay.n_seqs), want_rows=view(lay.want_rows, lay.n_want),
        page_tables=tables, max_new_tokens=max_new_tokens, max_ctx_len=max_ctx_len, is_decode=is_decode,
        new_tokens_host=new_tokens_host if new_tokens_host is not None else ([1] * lay.n_seqs if is_decode else None))
