"""Configuration and registry."""
import json

import pytest

import wpc_engine_b200 as wpc
from conftest import TINY_A, TINY_B, TINY_C
from wpc_engine_b200.config import ConfigError, Qwen2Config
from wpc_engine_b200.registry import config_from_folder, resolve


def test_reads_its_own_keys_and_ignores_others():
    cfg = Qwen2Config.from_dict(dict(TINY_A, some_unknown_key=[1, 2], torch_dtype="bfloat16"))
    assert (cfg.hidden_size, cfg.num_hidden_layers, cfg.head_dim, cfg.vocab_size) == (64, 2, 16, 256)
    assert cfg.tie_word_embeddings is True and cfg.window_of_layer(1) is None


def test_defaults():
    raw = {k: v for k, v in TINY_A.items() if k not in ("tie_word_embeddings", "max_position_embeddings")}
    cfg = Qwen2Config.from_dict(raw)
    assert cfg.tie_word_embeddings is True          # wpc-runtime/src/config.rs:18-19
    assert cfg.head_dim == 64 // 4                  # config.rs:59-62
    assert cfg.max_position_embeddings is None and cfg.eos_token_id == ()


def test_stated_head_dim_wins():
    cfg = Qwen2Config.from_dict(TINY_C)
    assert cfg.head_dim == 48 and cfg.q_size == 192 and cfg.kv_size == 96
    assert [cfg.window_of_layer(i) for i in range(3)] == [None, 40, 40]
    assert cfg.eos_token_id == (7, 9)


@pytest.mark.parametrize("key", ["vocab_size", "hidden_size", "num_hidden_layers", "num_attention_heads",
                                 "num_key_value_heads", "intermediate_size", "rope_theta", "rms_norm_eps"])
def test_missing_required_key_is_named(key):
    raw = {k: v for k, v in TINY_B.items() if k != key}
    with pytest.raises(ConfigError, match=key):
        Qwen2Config.from_dict(raw)


@pytest.mark.parametrize("change,word", [
    ({"num_key_value_heads": 2}, "multiple"), ({"hidden_size": 100}, "head_dim"),
    ({"rms_norm_eps": 0}, "rms_norm_eps"), ({"rope_theta": -1.0}, "rope_theta"),
    ({"vocab_size": 0}, "vocab_size"), ({"num_hidden_layers": 2.5}, "integer"),
    ({"head_dim": 31}, "even"), ({"use_sliding_window": True}, "sliding_window"),
    ({"eos_token_id": "x"}, "eos_token_id"), ({"tie_word_embeddings": "yes"}, "tie_word_embeddings"),
])
def test_bad_values_are_refused(change, word):
    with pytest.raises(ConfigError, match=word):
        Qwen2Config.from_dict(dict(TINY_B, **change))


def test_registry_resolves_by_architecture_then_model_type():
    assert resolve({"architectures": ["Qwen2ForCausalLM"]}).name == "Qwen2ForCausalLM"
    assert resolve({"model_type": "qwen2"}).name == "Qwen2ForCausalLM"
    with pytest.raises(ConfigError, match="unknown architecture"):
        resolve({"architectures": ["LlamaForCausalLM"], "model_type": "qwen2"})
    with pytest.raises(ConfigError, match="no known architecture"):
        resolve({"model_type": "qwen3"})         # no silent fallback to Qwen2


def test_round_trip_through_a_folder(tmp_path):
    cfg = Qwen2Config.from_dict(TINY_C)
    (tmp_path / "config.json").write_text(json.dumps(cfg.to_dict()))
    arch, back = config_from_folder(str(tmp_path))
    assert arch.name == "Qwen2ForCausalLM" and back == cfg
    with pytest.raises(ConfigError, match="no config.json"):
        config_from_folder(str(tmp_path / "nowhere"))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="not JSON"):
        config_from_folder(str(tmp_path))


def test_model_is_built_from_the_configuration_layer_by_layer():
    model = resolve(TINY_C).build(Qwen2Config.from_dict(TINY_C))
    assert len(model.blocks) == 3 and [r.layer for r in model.schedule] == [0, 1, 2]
    assert [b.mixer.window for b in model.blocks] == [None, 40, 40]
    assert model.blocks[0].mixer.position is model.blocks[2].mixer.position
    specs = model.cache_specs()
    assert specs[0] != specs[1] and specs[1] == specs[2]
    names = set(model.wanted_tensors())
    assert "lm_head.weight" in names and "model.layers.2.self_attn.k_proj.bias" in names
    tied = resolve(TINY_A).build(Qwen2Config.from_dict(TINY_A))
    assert "lm_head.weight" not in tied.wanted_tensors() and tied.ignored == ("lm_head.weight",)
