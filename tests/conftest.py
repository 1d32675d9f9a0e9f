"""Shared test set-up: the `gpu` marker, the tiny configurations, model folders made in a
temporary folder, and the CPU stand-ins for the device operations (tests/torch_ops.py) that
let the host-side logic of the engine run where there is no GPU."""
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import wpc_engine_b200 as wpc  # noqa: E402


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


# Tiny configurations that differ in every size and option.
TINY_A = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", num_hidden_layers=2, hidden_size=64,
              num_attention_heads=4, num_key_value_heads=2, intermediate_size=128, vocab_size=256,
              rope_theta=10000.0, rms_norm_eps=1e-6, max_position_embeddings=128,
              use_sliding_window=False, tie_word_embeddings=True)
TINY_B = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", num_hidden_layers=3, hidden_size=96,
              num_attention_heads=3, num_key_value_heads=1, intermediate_size=200, vocab_size=384,
              rope_theta=1000000.0, rms_norm_eps=1e-5, max_position_embeddings=256,
              use_sliding_window=False, tie_word_embeddings=False)
# stated head_dim that is not hidden/heads, a window on the layers after the first, odd vocabulary
TINY_C = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", num_hidden_layers=3, hidden_size=80,
              num_attention_heads=4, num_key_value_heads=2, head_dim=48, intermediate_size=136, vocab_size=300,
              rope_theta=500000.0, rms_norm_eps=1e-5, max_position_embeddings=1024,
              use_sliding_window=True, sliding_window=40, max_window_layers=1, tie_word_embeddings=False,
              eos_token_id=[7, 9])
TINY = {"A": (TINY_A, 0), "B": (TINY_B, 1), "C": (TINY_C, 2)}


def make_folder(tmp_path_factory, raw, seed, dtype, **override):
    raw = dict(raw, **override)
    cfg = wpc.Qwen2Config.from_dict(raw)
    folder = str(tmp_path_factory.mktemp("model"))
    wpc.write_random_model(folder, cfg, seed, dtype)
    return folder


@pytest.fixture(scope="session")
def folders(tmp_path_factory):
    """{(name, 'float32' | 'bfloat16'): model folder}, made on first use."""
    made = {}

    class Lazy(dict):
        def __missing__(self, key):
            name, dtype = key
            raw, seed = TINY[name]
            made[key] = make_folder(tmp_path_factory, raw, seed, getattr(torch, dtype))
            self[key] = made[key]
            return made[key]
    return Lazy()


@pytest.fixture
def cpu_ops(monkeypatch):
    """Replaces every device operation by its plain torch stand-in, so that the engine's host
    logic (cache, batching, generation) can run on the CPU.  Test-only: the package itself has
    no such path."""
    import torch_ops
    from wpc_engine_b200 import ops
    for name in torch_ops.__all__:
        monkeypatch.setattr(ops, name, getattr(torch_ops, name))
    return torch_ops
