"""Parts that layers are put together from; see base.py for the interfaces."""
from .attention import GQAAttention
from .base import (Block, FeedForward, HeadNorm, KVSpec, Mixer, Norm, ParamSpec, Part, PositionEncoding,
                   StateSpec, all_graph_safe, collect_params)
from .block import PreNormBlock
from .embedding import Embedding, OutputHead
from .linear import Linear, fuse_rows
from .mlp import GatedMLP, SwiGLU
from .norm import HeadRMSNorm, RMSNorm
from .rope import RotaryEncoding

__all__ = ["Block", "Embedding", "FeedForward", "GQAAttention", "GatedMLP", "HeadNorm", "HeadRMSNorm", "KVSpec",
           "Linear", "Mixer", "Norm", "OutputHead", "ParamSpec", "Part", "PositionEncoding", "PreNormBlock",
           "RMSNorm", "RotaryEncoding", "StateSpec", "SwiGLU", "all_graph_safe", "collect_params", "fuse_rows"]
