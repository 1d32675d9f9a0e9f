"""The Qwen2 dense decoder, assembled from parts (wpc-runtime/src/model.rs:64-117, 419-547).

Per layer: RMSNorm -> attention with q/k/v biases and rotary positions -> residual,
RMSNorm -> SwiGLU -> residual; tensor names as stored by the checkpoints
(model.rs:70, 80-94, 114).  The output head is the embedding table when
`tie_word_embeddings` holds, else `lm_head.weight`.
"""
from __future__ import annotations

from ..config.qwen2 import Qwen2Config
from ..parts import (Embedding, GQAAttention, OutputHead, PreNormBlock, RMSNorm, RotaryEncoding,
                     SwiGLU)
from .decoder import DecoderModel


def build_qwen2(config: Qwen2Config) -> DecoderModel:
    c = config
    rotary = RotaryEncoding(c.head_dim, c.rope_theta)          # shared by all layers
    blocks = []
    for layer in range(c.num_hidden_layers):
        blocks.append(PreNormBlock(
            RMSNorm(c.hidden_size, c.rms_norm_eps),
            GQAAttention(c.hidden_size, c.num_attention_heads, c.num_key_value_heads, c.head_dim,
                         position=rotary, qkv_bias=True, window=c.window_of_layer(layer)),
            RMSNorm(c.hidden_size, c.rms_norm_eps),
            SwiGLU(c.hidden_size, c.intermediate_size)))
    embedding = Embedding(c.vocab_size, c.hidden_size)
    head = OutputHead(c.vocab_size, c.hidden_size, tied_to=embedding if c.tie_word_embeddings else None)
    ignored = ("lm_head.weight",) if c.tie_word_embeddings else ()
    return DecoderModel(c, embedding, blocks, RMSNorm(c.hidden_size, c.rms_norm_eps), head, ignored=ignored,
                        max_positions=c.max_position_embeddings)
