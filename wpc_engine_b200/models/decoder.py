"""A decoder as data: parts, and the order in which the layers run.

Nothing here knows an architecture: a builder (see qwen2.py) makes the parts from a
configuration and names where their tensors are stored.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..cache import KVGroup, KVView, SequenceCache, StateGroup, StateView
from ..parts.base import Block, Norm, Part, all_graph_safe, collect_params
from ..parts.embedding import Embedding, OutputHead


@dataclass(frozen=True)
class Run:
    """One entry of the schedule: run block `layer`; with `cache_of` set, read the cache that
    the earlier schedule entry of that index wrote instead of keeping one of its own."""
    layer: int
    cache_of: Optional[int] = None


class DecoderModel:
    """embedding -> the scheduled blocks on the float32 residual stream -> final norm of the
    wanted rows -> output head (wpc-runtime/src/model.rs:419-547, for many tokens at once).

    `names` gives the stored-name prefix of each root part; `ignored` lists stored names that
    may be present without being used.  `max_positions`: the longest sequence that the model
    may see (None: no limit); the builder takes it from whatever key its configuration has.
    """

    def __init__(self, config, embedding: Embedding, blocks: Sequence[Block], final_norm: Norm,
                 head: OutputHead, schedule: Optional[Sequence[Run]] = None,
                 names: Optional[Dict[str, str]] = None, ignored: Sequence[str] = (),
                 max_positions: Optional[int] = None):
        self.config = config
        self.max_positions = None if max_positions is None else int(max_positions)
        self.embedding = embedding
        self.blocks = list(blocks)
        self.final_norm = final_norm
        self.head = head
        self.schedule = list(schedule) if schedule is not None else [Run(i) for i in range(len(self.blocks))]
        self.names = {"embedding": "model.embed_tokens", "blocks": "model.layers.{}",
                      "final_norm": "model.norm", "head": "lm_head"}
        self.names.update(names or {})
        self.ignored = tuple(ignored)
        for i, run in enumerate(self.schedule):
            if not 0 <= run.layer < len(self.blocks):
                raise ValueError(f"schedule entry {i} names layer {run.layer} of {len(self.blocks)}")
            if run.cache_of is not None:
                if not 0 <= run.cache_of < i or self.schedule[run.cache_of].cache_of is not None:
                    raise ValueError(f"schedule entry {i} reads the cache of entry {run.cache_of}, "
                                     "which is not an earlier entry with a cache of its own")

    @property
    def vocab_size(self) -> int:
        """Token ids that a step may bring: 0 .. vocab_size - 1."""
        return self.embedding.vocab_size

    # -- tensors -----------------------------------------------------------------------------
    def roots(self) -> List[Tuple[str, Part]]:
        out = [(self.names["embedding"], self.embedding)]
        out += [(self.names["blocks"].format(i), b) for i, b in enumerate(self.blocks)]
        out += [(self.names["final_norm"], self.final_norm), (self.names["head"], self.head)]
        return out

    def wanted_tensors(self):
        """full stored name -> (owning part, local name, ParamSpec)"""
        wanted = {}
        for prefix, part in self.roots():
            wanted.update(collect_params(part, prefix + "."))
        return wanted

    def graph_safe(self) -> bool:
        return all(all_graph_safe(part) for _, part in self.roots())

    # -- cache -------------------------------------------------------------------------------
    def cache_specs(self) -> List[object]:
        """What each schedule entry keeps per sequence (None for entries that keep nothing or
        read another entry's cache)."""
        specs = []
        for run in self.schedule:
            mixer = self.blocks[run.layer].mixer_of()
            own = run.cache_of is None and mixer is not None
            specs.append(mixer.cache_spec() if own else None)
        return specs

    def cache_views(self, cache: SequenceCache, ctx) -> List[object]:
        views: List[object] = []
        kv_order = cache.kv_groups()
        for i, run in enumerate(self.schedule):
            src = i if run.cache_of is None else run.cache_of
            g = cache.layer_group[src]
            if g is None:
                views.append(None)
                continue
            group, j = cache.groups[g], cache.layer_index[src]
            if isinstance(group, KVGroup):
                views.append(KVView(group.k[j], group.v[j], ctx.page_tables[kv_order.index(g)],
                                    writes=run.cache_of is None))
            elif isinstance(group, StateGroup):
                views.append(StateView(group.state[j], ctx.slots, writes=run.cache_of is None))
        return views

    # -- the forward pass of one step ----------------------------------------------------------
    def forward(self, ctx, cache: SequenceCache) -> Optional[torch.Tensor]:
        """Runs the step's tokens; returns float32 logits [n_want, vocab] (None if none wanted)."""
        views = self.cache_views(cache, ctx)
        x = self.embedding.forward(ctx)
        for run, view in zip(self.schedule, views):
            self.blocks[run.layer].forward(ctx, x, view)
        if ctx.want_rows.numel() == 0:
            return None
        h = self.final_norm.forward_rows(ctx, x, ctx.want_rows)
        return self.head.forward(ctx, h)
