"""The arrangement of parts in a layer."""
from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from .base import Block, FeedForward, Mixer, Norm


class PreNormBlock(Block):
    """x += mixer(norm1(x)); x += ffn(norm2(x))  (wpc-runtime/src/model.rs:432-536).

    The parts' names in the weights are parameters, since architectures name them
    differently.
    """

    def __init__(self, mixer_norm: Norm, mixer: Mixer, ffn_norm: Norm, ffn: FeedForward,
                 names=("input_layernorm", "self_attn", "post_attention_layernorm", "mlp")):
        self.mixer_norm = mixer_norm
        self.mixer = mixer
        self.ffn_norm = ffn_norm
        self.ffn = ffn
        self.names = tuple(names)

    def subparts(self) -> Dict[str, object]:
        return dict(zip(self.names, (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn)))

    def mixer_of(self):
        return self.mixer

    def forward(self, ctx, x: torch.Tensor, cache) -> None:
        h = self.mixer_norm.forward(ctx, x)
        y = self.mixer.forward(ctx, h, cache, x)
        if y is not None:
            ops.add_(x, y)
        h = self.ffn_norm.forward(ctx, x)
        y = self.ffn.forward(ctx, h, x)
        if y is not None:
            ops.add_(x, y)
