"""The engine's host logic (cache, batching, step, generation) on the CPU, with the device
operations replaced by their plain torch stand-ins, compared with the plain implementation."""
import numpy as np
import pytest

from helpers import (assert_close_to_plain, plain_logits, random_tokens, run_batch, run_tail_one_by_one,
                     run_whole)
from plain import qwen2_plain as P
from wpc_engine_b200 import Engine, GenerationOptions, generate


def cpu_engine(folder, **kw):
    kw.setdefault("max_tokens", 2048)
    return Engine.from_folder(folder, dtype="float32", device="cpu", **kw)


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_whole_chunked_and_batched_agree_with_plain(cpu_ops, folders, name):
    folder = folders[(name, "float32")]
    eng = cpu_engine(folder)
    vocab = eng.config.vocab_size
    reqs = [random_tokens(vocab, n, 10 + i) for i, n in enumerate([70, 5, 33, 100])]
    for r in reqs:
        assert_close_to_plain(run_whole(eng, r), folder, r, "float32", "whole")
        assert_close_to_plain(run_tail_one_by_one(eng, r), folder, r, "float32", "tail one by one")
    for round_ in range(2):          # twice: the second batch reuses the slots of the first
        outs = run_batch(eng, reqs, [20, 5, 1, 64])
        for r, o in zip(reqs, outs):
            assert_close_to_plain(o, folder, r, "float32", f"batch round {round_}")
    eng.cache.check()
    assert eng.cache.slots.n_held == 0
    assert all(g.pool.n_held == 0 for g in eng.cache.groups if hasattr(g, "pool"))


def test_generation_matches_plain_greedy(cpu_ops, folders):
    folder = folders[("A", "float32")]
    eng = cpu_engine(folder)
    cfg, tensors = P.read_model_folder(folder)
    prompts = [random_tokens(256, n, 40 + n) for n in (5, 11, 17)]
    got = generate(eng, prompts, GenerationOptions(max_tokens=8))
    for p, g in zip(prompts, got):
        assert g == P.generate_greedy(cfg, tensors, p, 8)
    eng.cache.check()
    assert eng.cache.slots.n_held == 0
