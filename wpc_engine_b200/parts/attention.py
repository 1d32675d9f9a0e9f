"""Grouped-query attention over the paged cache (wpc-runtime/src/model.rs:437-516)."""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from .. import ops
from .base import HeadNorm, KVSpec, Mixer, PositionEncoding
from .linear import Linear, fuse_rows


class GQAAttention(Mixer):
    """q, k, v projections (with or without bias), position encoding on q and k, keys (after
    rotation, model.rs:471-475) and values appended to the cache, softmax(q.k * scale) over
    the visible positions, weighted values, output projection without bias added to the
    residual stream.

    Query head qh reads KV head qh // (n_heads // n_kv_heads) (model.rs:484).  `window`
    None: a query sees every earlier position and itself; else only the last `window`.
    `scale` None: 1/sqrt(head_dim) (model.rs:477).  `q_norm`, `k_norm`: norms of each head
    of q and of k between projection and position encoding (model.rs:447-462; the Qwen2
    layers have none).  All sizes are parameters.

    With a position encoding that rotates half-split pairs and no head norms, one kernel does
    the projection, the rotation and the cache write; otherwise these run one after another
    (projection, head norms, `position.rotate`, cache write), with the same result.
    """

    def __init__(self, width: int, n_heads: int, n_kv_heads: int, head_dim: int,
                 position: Optional[PositionEncoding], qkv_bias: bool = True,
                 window: Optional[int] = None, scale: Optional[float] = None,
                 names=("q_proj", "k_proj", "v_proj", "o_proj"),
                 q_norm: Optional[HeadNorm] = None, k_norm: Optional[HeadNorm] = None,
                 norm_names=("q_norm", "k_norm")):
        if n_heads % n_kv_heads:
            raise ValueError(f"n_heads {n_heads} is not a multiple of n_kv_heads {n_kv_heads}")
        self.width = int(width)
        self.n_heads = int(n_heads)
        self.n_kv_heads = int(n_kv_heads)
        self.head_dim = int(head_dim)
        self.position = position
        self.window = None if window is None else int(window)
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.head_dim)
        self.q_proj = Linear(width, n_heads * head_dim, bias=qkv_bias)
        self.k_proj = Linear(width, n_kv_heads * head_dim, bias=qkv_bias)
        self.v_proj = Linear(width, n_kv_heads * head_dim, bias=qkv_bias)
        self.o_proj = Linear(n_heads * head_dim, width, bias=False)
        self.names = tuple(names)
        self.q_norm, self.k_norm = q_norm, k_norm
        self.norm_names = tuple(norm_names)
        self.qkv = None

    def subparts(self) -> Dict[str, object]:
        subs = dict(zip(self.names, (self.q_proj, self.k_proj, self.v_proj, self.o_proj)))
        for name, norm in zip(self.norm_names, (self.q_norm, self.k_norm)):
            if norm is not None:
                subs[name] = norm
        return subs

    def cache_spec(self):
        return KVSpec(self.n_kv_heads, self.head_dim, self.window)

    def finalize(self):
        self.qkv = fuse_rows([self.q_proj, self.k_proj, self.v_proj])
        nq = self.n_heads * self.head_dim
        nk = self.n_kv_heads * self.head_dim
        w, b = self.qkv.weight, self.qkv.bias
        for lin, lo, hi in ((self.q_proj, 0, nq), (self.k_proj, nq, nq + nk), (self.v_proj, nq + nk, nq + 2 * nk)):
            lin.weight = w[lo:hi]
            lin.bias = None if b is None else b[lo:hi]

    def _fused(self) -> bool:
        """Whether one kernel may project, rotate and write the cache: its tail knows half-split
        rotation by (cos, sin) tables and nothing between projection and rotation."""
        plain_rotation = self.position is None or (self.position.pairing == "half_split"
                                                   and type(self.position).rotate is PositionEncoding.rotate)
        return plain_rotation and self.q_norm is None and self.k_norm is None

    def forward(self, ctx, h: torch.Tensor, cache, residual: torch.Tensor):
        nh, nkv, hd = self.n_heads, self.n_kv_heads, self.head_dim
        if cache.writes and self._fused():
            cos = sin = None
            if self.position is not None:
                cos, sin = self.position.tables(ctx)
            qkv = ops.linear_qk_rope_kv_store(h, self.qkv.weight, self.qkv.bias, nh, nkv, hd, cos, sin,
                                              cache.k_pages, cache.v_pages, cache.page_table,
                                              ctx.seq_of_token, ctx.positions)
        else:
            # step by step; a layer that reads another layer's cache computes queries only
            qkv = self.qkv.forward(h) if cache.writes else self.q_proj.forward(h)
            if self.q_norm is not None:
                self.q_norm.forward_heads(ctx, qkv, nh, hd)
            if self.k_norm is not None and cache.writes:
                self.k_norm.forward_heads(ctx, qkv[:, nh * hd:], nkv, hd)
            if self.position is not None:       # the k heads lie right behind the q heads
                self.position.rotate(ctx, qkv, nh + nkv if cache.writes else nh, hd)
            if cache.writes:
                ops.qk_rope_kv_store(qkv, nh, nkv, hd, None, None, cache.k_pages, cache.v_pages, cache.page_table,
                                     ctx.seq_of_token, ctx.positions)
        attn = ops.attention(qkv, nh, nkv, hd, cache.k_pages, cache.v_pages, cache.page_table,
                             ctx.cu_seqlens, ctx.ctx_lens, ctx.seq_of_token, ctx.positions,
                             self.scale, self.window, ctx.max_new_tokens, ctx.max_ctx_len)
        self.o_proj.forward(attn, residual=residual)
        return None
