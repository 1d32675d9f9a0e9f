"""Token embedding and output head (wpc-runtime/src/weights.rs:25-31, 94-121)."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import ops
from .base import ParamSpec, Part


class Embedding(Part):
    """x = table[token] (a row copy, no scaling; weights.rs:101-105), into the float32
    residual stream."""

    def __init__(self, vocab_size: int, width: int):
        self.vocab_size = int(vocab_size)
        self.width = int(width)
        self.table = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {"weight": ParamSpec((self.vocab_size, self.width), kind="table")}

    def bind(self, tensors):
        self.table = tensors["weight"]

    def forward(self, ctx) -> torch.Tensor:
        return ops.embed(ctx.tokens, self.table)


class OutputHead(Part):
    """logits = table . x in float32 (weights.rs:106-120).  With `tied_to` the table is the
    embedding's (the reference's only case, model.rs:544-546); else a matrix of its own."""

    def __init__(self, vocab_size: int, width: int, tied_to: Optional[Embedding] = None):
        self.vocab_size = int(vocab_size)
        self.width = int(width)
        self.tied_to = tied_to
        self.table = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        if self.tied_to is not None:
            return {}
        return {"weight": ParamSpec((self.vocab_size, self.width), kind="matrix")}

    def bind(self, tensors):
        self.table = tensors.get("weight")

    def forward(self, ctx, h: torch.Tensor) -> torch.Tensor:
        table = self.tied_to.table if self.tied_to is not None else self.table
        return ops.linear(h, table, None, out_dtype=torch.float32, static_weight=True)
