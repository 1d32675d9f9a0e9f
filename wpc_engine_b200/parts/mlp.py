"""Gated feed-forward with SiLU (wpc-runtime/src/model.rs:518-536)."""
from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from .base import FeedForward
from .linear import Linear, fuse_rows


class SwiGLU(FeedForward):
    """down( silu(gate(h)) * up(h) ), no biases (model.rs:107-109).

    After loading, the gate and up matrices are stacked into one [2*inner, width] matrix so
    that one product reads h once; the activation reads both halves of a row.
    """

    def __init__(self, width: int, inner: int):
        self.width = int(width)
        self.inner = int(inner)
        self.gate_proj = Linear(width, inner)
        self.up_proj = Linear(width, inner)
        self.down_proj = Linear(inner, width)
        self.gate_up = None

    def subparts(self) -> Dict[str, object]:
        return {"gate_proj": self.gate_proj, "up_proj": self.up_proj, "down_proj": self.down_proj}

    def finalize(self):
        self.gate_up = fuse_rows([self.gate_proj, self.up_proj])
        self.gate_proj.weight = self.gate_up.weight[: self.inner]
        self.up_proj.weight = self.gate_up.weight[self.inner:]

    def forward(self, ctx, h: torch.Tensor, residual: torch.Tensor):
        gu = self.gate_up.forward(h)
        act = ops.silu_mul(gu, self.inner)
        self.down_proj.forward(act, residual=residual)
        return None
