"""Root-mean-square norm with a learned gain (wpc-runtime/src/norm.rs:4-13)."""
from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from .base import Norm, ParamSpec


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
