"""Typed configuration of the Qwen2 dense decoder, read from its own config.json keys.

Required and optional keys and the two defaults follow the reference's `Config`
(wpc-runtime/src/config.rs:8-62): `tie_word_embeddings` defaults to true (config.rs:18-19)
and `head_dim` to hidden_size / num_attention_heads (config.rs:59-62).  The window keys
(`sliding_window`, `use_sliding_window`, `max_window_layers`) and `max_position_embeddings`
are not read by the reference; here they mean what their names say: with
`use_sliding_window` set, layers `max_window_layers` and above see only the last
`sliding_window` positions, and no sequence may grow beyond `max_position_embeddings`.
"""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .base import ConfigError, from_keys, require, require_int, require_number


@dataclass(frozen=True)
class Qwen2Config:
    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    intermediate_size: int
    rope_theta: float
    rms_norm_eps: float
    tie_word_embeddings: bool = True
    head_dim: Optional[int] = None
    max_position_embeddings: Optional[int] = None
    sliding_window: Optional[int] = None
    use_sliding_window: bool = False
    max_window_layers: Optional[int] = None
    eos_token_id: Any = None          # a number or a list of numbers (main.rs:449-488)
    bos_token_id: Optional[int] = None
    model_type: Optional[str] = None
    architectures: Tuple[str, ...] = ()

    ARCHITECTURE = "Qwen2ForCausalLM"

    def __post_init__(self):
        for name in ("vocab_size", "hidden_size", "num_hidden_layers", "num_attention_heads",
                     "num_key_value_heads", "intermediate_size"):
            require_int(name, getattr(self, name))
        object.__setattr__(self, "rope_theta", require_number("rope_theta", self.rope_theta))
        object.__setattr__(self, "rms_norm_eps", require_number("rms_norm_eps", self.rms_norm_eps))
        require(self.rope_theta > 0, f"rope_theta must be > 0, got {self.rope_theta}")
        require(self.rms_norm_eps > 0, f"rms_norm_eps must be > 0, got {self.rms_norm_eps}")
        require(isinstance(self.tie_word_embeddings, bool), "tie_word_embeddings must be true or false")
        require(isinstance(self.use_sliding_window, bool), "use_sliding_window must be true or false")
        require(self.num_attention_heads % self.num_key_value_heads == 0,
                f"num_attention_heads ({self.num_attention_heads}) must be a multiple of "
                f"num_key_value_heads ({self.num_key_value_heads})")
        if self.head_dim is None:
            require(self.hidden_size % self.num_attention_heads == 0,
                    f"hidden_size ({self.hidden_size}) is not a multiple of num_attention_heads "
                    f"({self.num_attention_heads}) and head_dim is not given")
            object.__setattr__(self, "head_dim", self.hidden_size // self.num_attention_heads)
        require_int("head_dim", self.head_dim)
        require(self.head_dim % 2 == 0, f"head_dim must be even for the rotation, got {self.head_dim}")
        if self.max_position_embeddings is not None:
            require_int("max_position_embeddings", self.max_position_embeddings)
        if self.sliding_window is not None:
            require_int("sliding_window", self.sliding_window)
        if self.max_window_layers is not None:
            require_int("max_window_layers", self.max_window_layers, minimum=0)
        if self.use_sliding_window:
            require(self.sliding_window is not None, "use_sliding_window is set but sliding_window is not given")
        eos = self.eos_token_id
        if eos is None:
            eos = ()
        elif isinstance(eos, int) and not isinstance(eos, bool):
            eos = (eos,)
        elif isinstance(eos, (list, tuple)) and all(isinstance(e, int) and not isinstance(e, bool) for e in eos):
            eos = tuple(sorted(set(eos)))
        else:
            raise ConfigError(f"eos_token_id must be a number or a list of numbers, got {self.eos_token_id!r}")
        object.__setattr__(self, "eos_token_id", eos)
        object.__setattr__(self, "architectures", tuple(self.architectures or ()))

    # -- derived -------------------------------------------------------------------------
    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    def window_of_layer(self, layer: int) -> Optional[int]:
        """The window of `layer`, or None when it sees every earlier position."""
        if not self.use_sliding_window or self.sliding_window is None:
            return None
        return self.sliding_window if layer >= (self.max_window_layers or 0) else None

    # -- reading and writing -----------------------------------------------------------------
    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "Qwen2Config":
        return from_keys(cls, raw)

    def to_dict(self) -> Dict[str, Any]:
        """The config.json of this configuration (what the random-weights mode writes)."""
        d = {f.name: getattr(self, f.name) for f in dataclasses.fields(self)}
        d["architectures"] = list(self.architectures) or [self.ARCHITECTURE]
        d["model_type"] = self.model_type or "qwen2"
        eos = d.pop("eos_token_id")
        if len(eos) == 1:
            d["eos_token_id"] = eos[0]
        elif len(eos) > 1:
            d["eos_token_id"] = list(eos)
        return {k: v for k, v in d.items() if v is not None}
