"""Rotary position encoding, half-split pairs (wpc-runtime/src/rope.rs:10-40)."""
from __future__ import annotations

import numpy as np
import torch

from .. import ops
from .base import PositionEncoding


class RotaryEncoding(PositionEncoding):
    """Rotates the pairs (i, i + head_dim/2) of a head by pos * theta^(-2i/head_dim).

    `rotary_pairs` may be smaller than head_dim/2: the remaining pairs then pass through
    (rope.rs:24-40).  The inverse frequencies are computed here on the host in float64, as
    rope.rs:30 does; each step multiplies them by the step's positions and takes sine and
    cosine in float64 on the device (rope.rs:31-33), once for all layers that share this
    object.
    """

    def __init__(self, head_dim: int, theta: float, rotary_pairs: int | None = None):
        self.head_dim = int(head_dim)
        self.theta = float(theta)
        self.rotary_pairs = self.head_dim // 2 if rotary_pairs is None else int(rotary_pairs)
        if not 0 < self.rotary_pairs <= self.head_dim // 2:
            raise ValueError(f"rotary_pairs {self.rotary_pairs} outside 1..{self.head_dim // 2}")
        i = np.arange(self.rotary_pairs, dtype=np.float64)
        self._inv_freq_host = np.power(np.float64(self.theta), -(2.0 * i) / np.float64(self.head_dim))
        self._inv_freq = None

    def inv_freq(self, device) -> torch.Tensor:
        if self._inv_freq is None or self._inv_freq.device != torch.device(device):
            self._inv_freq = torch.from_numpy(self._inv_freq_host.copy()).to(device)
        return self._inv_freq

    def tables(self, ctx):
        """(cos, sin), float32 [T, rotary_pairs], for the positions of this step."""
        key = ("rotary", id(self))
        got = ctx.shared.get(key)
        if got is None:
            got = ops.rope_angles(ctx.positions, self.inv_freq(ctx.positions.device))
            ctx.shared[key] = got
        return got
