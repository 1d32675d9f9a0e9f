"""y = x W^T (+ b): the one place where a matrix product is chosen
(wpc-runtime/src/weights.rs:17-22, 59-78: `W` is [out, in] row-major, the bias is added
after the dot product)."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import ops
from .base import ParamSpec, Part


class Linear(Part):
    def __init__(self, in_features: int, out_features: int, bias: bool = False):
        self.in_features = int(in_features)
        self.out_features = int(out_features)
        self.has_bias = bool(bias)
        self.weight = None
        self.bias = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        specs = {"weight": ParamSpec((self.out_features, self.in_features), kind="matrix")}
        if self.has_bias:
            specs["bias"] = ParamSpec((self.out_features,), kind="vector")
        return specs

    def bind(self, tensors):
        self.weight = tensors["weight"]
        self.bias = tensors.get("bias")

    def forward(self, x: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
                residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        """With `residual` (float32 [T, out]) the product is added to it in place, in float32,
        and `residual` is returned; else a new [T, out] tensor of `out_dtype` (default x's)."""
        return ops.linear(x, self.weight, self.bias, out_dtype=out_dtype, residual=residual, static_weight=True)


def fuse_rows(parts):
    """One Linear whose weight is the rows of `parts` one below the other (a pure re-layout:
    each output row is computed exactly as before).  All must be bound and agree on bias."""
    first = parts[0]
    fused = Linear(first.in_features, sum(p.out_features for p in parts), bias=first.has_bias)
    tensors = {"weight": torch.cat([p.weight for p in parts], dim=0).contiguous()}
    if first.has_bias:
        tensors["bias"] = torch.cat([p.bias for p in parts], dim=0).contiguous()
    fused.bind(tensors)
    return fused
