"""Root-mean-square norm with a learned gain (wpc-runtime/src/norm.rs:4-13)."""
from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from .base import HeadNorm, Norm, ParamSpec


class RMSNorm(Norm):
    """out = x * rsqrt(mean(x^2) + eps) * gain, statistics in float32.

    width and eps are parameters; the gain is plain `w` (not 1 + w), as in norm.rs:11.
    """

    def __init__(self, width: int, eps: float):
        self.width = int(width)
        self.eps = float(eps)
        self.gain = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {"weight": ParamSpec((self.width,), kind="vector", init="gain")}

    def bind(self, tensors):
        self.gain = tensors["weight"]

    def forward(self, ctx, x: torch.Tensor) -> torch.Tensor:
        return ops.rmsnorm(x, self.gain, self.eps, ctx.act_dtype)

    def forward_rows(self, ctx, x: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
        return ops.rmsnorm(x, self.gain, self.eps, ctx.act_dtype, rows=rows)


class HeadRMSNorm(HeadNorm):
    """The same norm over each head of a row (width head_dim, one gain vector for all heads):
    the per-head norm of q and k between projection and rotation that the reference's layer
    has as an option (wpc-runtime/src/model.rs:14-21, 447-462)."""

    def __init__(self, head_dim: int, eps: float):
        self.head_dim = int(head_dim)
        self.eps = float(eps)
        self.gain = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {"weight": ParamSpec((self.head_dim,), kind="vector", init="gain")}

    def bind(self, tensors):
        self.gain = tensors["weight"]

    def forward_heads(self, ctx, x: torch.Tensor, n_heads: int, head_dim: int) -> None:
        if head_dim != self.head_dim:
            raise ValueError(f"this norm is {self.head_dim} wide, the heads are {head_dim}")
        ops.head_rmsnorm_(x, n_heads, head_dim, self.gain, self.eps)
