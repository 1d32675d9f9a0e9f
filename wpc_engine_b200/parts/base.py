"""The interfaces that a layer is put together from.

A model is a list of blocks; a block arranges a mixer and a feed-forward around norms; a
mixer may use a position encoding and a cache.  Every part takes its sizes and constants as
constructor arguments and never looks at a model's configuration, so that one model can use
different parts in different layers and another architecture can reuse them.

What each kind of part must offer:

* every part: `param_specs()` (the tensors it wants, by local name, with shapes) and
  `bind(tensors)` (receives them on the device; may re-lay them out, bit-exactly).
* `Norm`:               `forward(ctx, x)`: x is the float32 residual stream [T, width];
                         returns the normed rows in the activation dtype.  Optional:
                         `forward_rows(ctx, x, rows)`, the same for the rows x[rows] only.
* `HeadNorm`:           `forward_heads(ctx, x, n_heads, head_dim)`: norms each of the first
                         n_heads heads of every row of x (activation dtype) in place.
* `PositionEncoding`:    `pairing` names which two elements of a head are rotated together:
                         "half_split" (i, i + head_dim/2) or "interleaved" (2i, 2i + 1);
                         `tables(ctx)`: (cos, sin), float32 [T, pairs], for this step's
                         positions, computed once a step and shared by all layers that hold
                         the same encoding object; `rotate(ctx, x, n_heads, head_dim)` applies
                         them in place (an encoding that is no rotation overrides it).
* `Mixer`:               `cache_spec()`: what it keeps per sequence (`KVSpec`, `StateSpec` or
                         None); `forward(ctx, h, cache, residual)`: h is [T, width] in the
                         activation dtype; it either adds its output to `residual` in place
                         and returns None, or returns [T, width] for the block to add.
* `FeedForward`:         `forward(ctx, h, residual)`, same contract as the mixer's.
* `Block`:               `forward(ctx, x, cache)`: runs its parts on the residual stream.

`ctx` is the step's `StepContext` (engine/batch.py): the packed tokens of all sequences of
the step, their positions and sequence numbers, and the page tables of each cache group.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import torch


@dataclass(frozen=True)
class ParamSpec:
    """A tensor that a part wants from the weights.

    kind: "matrix" (used in a matrix product: kept in the stored 16- or 32-bit type),
          "vector" (gains and biases: widened to float32, which is exact),
          "table"  (rows looked up by an integer id: kept like a matrix),
          "index"  (a table of integers: kept as int32).
    init: how the random-weights mode fills it: "normal" (N(0, 0.02)), "gain" (1 + N(0, 0.02));
          an "index" tensor is filled with integers drawn evenly from 0 .. high - 1 (zeros
          without `high`).
    """
    shape: Tuple[int, ...]
    kind: str = "matrix"
    init: str = "normal"
    high: Optional[int] = None


@dataclass(frozen=True)
class KVSpec:
    """Keys and values per position: `window` None keeps all of them, else the last `window`.
    `v_head_dim` None: values are as wide as keys (`head_dim`)."""
    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None
    v_head_dim: Optional[int] = None

    @property
    def value_dim(self) -> int:
        return self.head_dim if self.v_head_dim is None else self.v_head_dim


@dataclass(frozen=True)
class StateSpec:
    """A record of fixed size per sequence (for instance a recurrent state)."""
    shape: Tuple[int, ...]
    dtype: str = "float32"


class Part:
    # False for a part whose forward pass cannot be captured into a CUDA graph (it synchronises
    # with the host, or its launches depend on values that change from step to step); the
    # engine then runs the model's single-token steps directly.
    graph_safe = True

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {}

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        if tensors:
            raise ValueError(f"{type(self).__name__} takes no tensors, got {sorted(tensors)}")

    def subparts(self) -> Dict[str, "Part"]:
        """Parts that this part owns, by the name under which their tensors are stored."""
        return {}


class Norm(Part):
    def forward(self, ctx, x: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    def forward_rows(self, ctx, x: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
        """The norm of the rows x[rows] only (the places whose logits are wanted); a norm may
        override this to gather and norm in one kernel."""
        from .. import ops
        return self.forward(ctx, ops.gather_rows(x, rows))


class HeadNorm(Part):
    def forward_heads(self, ctx, x: torch.Tensor, n_heads: int, head_dim: int) -> None:
        raise NotImplementedError


class PositionEncoding(Part):
    pairing = "half_split"

    def tables(self, ctx):
        raise NotImplementedError

    def rotate(self, ctx, x: torch.Tensor, n_heads: int, head_dim: int) -> None:
        """Applies the encoding to the first n_heads heads of every row of x, in place."""
        from .. import ops
        if self.pairing not in ("half_split", "interleaved"):
            raise ValueError(f"{type(self).__name__}: pairing must be 'half_split' or 'interleaved', "
                             f"got {self.pairing!r}")
        cos, sin = self.tables(ctx)
        ops.rope_inplace(x, n_heads, head_dim, cos, sin, interleaved=self.pairing == "interleaved")


class Mixer(Part):
    def cache_spec(self):
        return None

    def forward(self, ctx, h: torch.Tensor, cache, residual: torch.Tensor) -> Optional[torch.Tensor]:
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, ctx, h: torch.Tensor, residual: torch.Tensor) -> Optional[torch.Tensor]:
        raise NotImplementedError


class Block(Part):
    def mixer_of(self) -> Optional[Mixer]:
        return None

    def forward(self, ctx, x: torch.Tensor, cache) -> None:
        raise NotImplementedError


def all_graph_safe(part: Part) -> bool:
    return bool(part.graph_safe) and all(all_graph_safe(sub) for sub in part.subparts().values())


def collect_params(part: Part, prefix: str = "") -> Dict[str, Tuple[Part, str, ParamSpec]]:
    """All tensors wanted below `part`: full name -> (owning part, local name, spec)."""
    out: Dict[str, Tuple[Part, str, ParamSpec]] = {}
    for local, spec in part.param_specs().items():
        out[prefix + local] = (part, local, spec)
    for name, sub in part.subparts().items():
        sub_prefix = prefix + name + "." if name else prefix
        for full, entry in collect_params(sub, sub_prefix).items():
            if full in out:
                raise ValueError(f"tensor name {full} is wanted twice")
            out[full] = entry
    return out
