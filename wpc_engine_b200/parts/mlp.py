"""Gated feed-forward (wpc-runtime/src/model.rs:518-536: with SiLU)."""
from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from .base import FeedForward
from .linear import Linear


class GatedMLP(FeedForward):
    """down( act(gate(h)) * up(h) ), no biases (model.rs:107-109).  `activation` is one of
    `ops.ACTIVATIONS` ("silu": the reference's, model.rs:527-531; "gelu_tanh").

    After loading, the gate and up matrices become one [2*inner, width] matrix so that one
    product reads h once.  Their rows are interleaved in blocks of `group` features (`group`
    gate rows, then the `group` up rows of the same features): with 16-bit weights and an
    inner size that 64 divides the group is 64, which lets the product's epilogue apply the
    activation; otherwise the group is the whole inner size (all gates, then all ups).  Each
    output is still the same dot product of the same row: a pure re-layout.
    """

    def __init__(self, width: int, inner: int, activation: str = "silu"):
        if activation not in ops.ACTIVATIONS:
            raise ValueError(f"unknown activation {activation!r}; known: {sorted(ops.ACTIVATIONS)}")
        self.activation = activation
        self.width = int(width)
        self.inner = int(inner)
        self.gate_proj = Linear(width, inner)
        self.up_proj = Linear(width, inner)
        self.down_proj = Linear(inner, width)
        self.gate_up = None
        self.group = self.inner

    def subparts(self) -> Dict[str, object]:
        return {"gate_proj": self.gate_proj, "up_proj": self.up_proj, "down_proj": self.down_proj}

    def finalize(self):
        g, u = self.gate_proj.weight, self.up_proj.weight
        G = ops.GATED_GROUP
        self.group = G if (self.inner % G == 0 and g.dtype == torch.bfloat16) else self.inner
        blocks = self.inner // self.group
        fused = torch.stack([g.view(blocks, self.group, self.width), u.view(blocks, self.group, self.width)], dim=1)
        self.gate_up = Linear(self.width, 2 * self.inner)
        self.gate_up.bind({"weight": fused.reshape(2 * self.inner, self.width).contiguous()})
        view = self.gate_up.weight.view(blocks, 2, self.group, self.width)
        self.gate_proj.weight, self.up_proj.weight = view[:, 0], view[:, 1]     # [blocks, group, width] views

    def forward(self, ctx, h: torch.Tensor, residual: torch.Tensor):
        act = ops.gated_linear(h, self.gate_up.weight, self.inner, self.group, static_weight=True,
                               activation=self.activation)
        self.down_proj.forward(act, residual=residual)
        return None


class SwiGLU(GatedMLP):
    """The gated feed-forward with SiLU, the reference's (model.rs:518-536)."""

    def __init__(self, width: int, inner: int):
        super().__init__(width, inner, "silu")
