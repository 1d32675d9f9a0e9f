"""The plain implementation against the anchor vectors of the reference's own unit tests and
against itself (float32 against float64)."""
import math

import numpy as np
import pytest

from conftest import TINY_A, TINY_C
from helpers import plain_logits, random_tokens
from plain import qwen2_plain as P


def test_rms_norm_anchor():
    # wpc-runtime/src/norm.rs:49-60 and 62-71
    out = P.rms_norm(np.array([3.0, 4.0, 0.0, 0.0], dtype=np.float32), np.ones(4, dtype=np.float32), 1e-6)
    assert np.allclose(out, [1.2, 1.6, 0.0, 0.0], atol=1e-4)
    out = P.rms_norm(np.ones(4, dtype=np.float32), np.array([2.0, 0.5, 1.0, 1.0], dtype=np.float32), 1e-6)
    assert np.allclose(out, [2.0, 0.5, 1.0, 1.0], atol=1e-4)


def test_softmax_anchor():
    # wpc-runtime/src/norm.rs:73-89
    p = P.softmax(np.array([1.0, 2.0, 3.0], dtype=np.float32))
    assert abs(p.sum() - 1.0) < 1e-6 and p[0] < p[1] < p[2]
    assert np.allclose(P.softmax(np.full(4, 5.0, dtype=np.float32)), 0.25)


def test_rope_anchor():
    # wpc-runtime/src/rope.rs:46-72: position 0 is the identity; pair norms are kept at position 5
    x = np.arange(1, 9, dtype=np.float32).reshape(1, 1, 8)
    assert np.array_equal(P.rope(x, [0], 1e6), x)
    y = P.rope(x, [5], 1e6)
    for i in range(4):
        assert math.isclose(x[0, 0, i] ** 2 + x[0, 0, i + 4] ** 2, y[0, 0, i] ** 2 + y[0, 0, i + 4] ** 2, rel_tol=1e-5)
    assert not np.allclose(x, y)


def test_argmax_anchor():
    # wpc-runtime/src/sampling.rs:57-74
    logits = [0.1, 5.0, -2.0, 4.9]
    assert P.argmax(logits) == 1
    assert P.argmax(logits, banned=[1]) == 3
    assert P.argmax(logits, banned=[1, 3]) == 0
    assert P.argmax([2.0, 2.0]) == 0 and P.argmax([]) == 0


def test_head_dim():
    # wpc-runtime/src/config.rs:140-160
    assert P.head_dim_of({"hidden_size": 1536, "num_attention_heads": 12}) == 128
    assert P.head_dim_of({"hidden_size": 2560, "num_attention_heads": 32, "head_dim": 128}) == 128


def test_float32_stays_close_to_float64(folders):
    folder = folders[("C", "float32")]
    toks = random_tokens(TINY_C["vocab_size"], 90, 3)
    a, b = plain_logits(folder, toks, np.float32), plain_logits(folder, toks, np.float64)
    assert np.abs(a - b).max() < 1e-4 * np.abs(b).max()


def test_prefix_logits_do_not_depend_on_later_tokens(folders):
    folder = folders[("A", "float32")]
    toks = random_tokens(TINY_A["vocab_size"], 40, 4)
    full, head = plain_logits(folder, toks), plain_logits(folder, toks[:17])
    assert np.allclose(full[:17], head, atol=1e-12)


def test_window_changes_only_late_positions(folders):
    folder = folders[("C", "float32")]
    cfg, tensors = P.read_model_folder(folder)
    toks = random_tokens(cfg["vocab_size"], 80, 5)
    windowed = P.forward(cfg, tensors, toks, np.float64)
    full = P.forward(dict(cfg, use_sliding_window=False), tensors, toks, np.float64)
    w = cfg["sliding_window"]
    assert np.allclose(windowed[:w], full[:w], atol=1e-12)
    assert np.abs(windowed[w + 5:] - full[w + 5:]).max() > 1e-6


def test_sampler_uniforms_and_cdf():
    us = [P.uniform_for(7, r, s) for r in range(4) for s in range(50)]
    assert all(0.0 <= u < 1.0 for u in us) and len(set(us)) == len(us)
    assert abs(np.mean(us) - 0.5) < 0.1
    idx, cdf, target = P.sample_temperature([0.0, math.log(3.0)], 1.0, 0.2)
    assert idx == 0 and P.sample_temperature([0.0, math.log(3.0)], 1.0, 0.3)[0] == 1
