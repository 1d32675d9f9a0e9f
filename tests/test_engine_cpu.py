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


def test_pipelined_loop_stops_at_the_longest_sequence_only_when_it_must(cpu_ops, folders):
    """The loop queues the next step before it has seen the tokens of this one.  A sequence that
    has no room for another token gets no such step; it is an error only if its last token turns
    out to be no stop token.  (On the CPU the loop runs with plain tensors in place of pinned
    memory and events.)"""
    folder = folders[("A", "float32")]           # at most 128 positions
    eng = cpu_engine(folder)
    eng.supports_device_tokens = True
    cfg, tensors = P.read_model_folder(folder)
    prompt = random_tokens(256, 126, 77)
    free = P.generate_greedy(cfg, tensors, prompt, 3)
    # 126 prompt tokens: the first two drawn tokens are fed (positions 126, 127), the third has no room
    assert generate(eng, [prompt], GenerationOptions(max_tokens=3)) == [free]
    if free[2] not in free[:2]:
        assert generate(eng, [prompt], GenerationOptions(max_tokens=9, stop_token_ids=[free[2]])) == [free]
    with pytest.raises(ValueError, match="longest sequence"):
        generate(eng, [prompt], GenerationOptions(max_tokens=9))
    assert eng.cache.slots.n_held == 0
    eng.cache.check()
    # a shorter request beside it goes on
    other = random_tokens(256, 5, 78)
    got = generate(eng, [prompt, other], GenerationOptions(max_tokens=3))
    assert got == [free, P.generate_greedy(cfg, tensors, other, 3)]


def test_pipelined_loop_reads_the_status_word_with_the_ids(cpu_ops, folders):
    import torch
    from wpc_engine_b200 import KernelError
    eng = cpu_engine(folders[("A", "float32")])
    eng.supports_device_tokens = True
    word = torch.zeros(1, dtype=torch.int32)
    eng.status_word = lambda: word
    assert len(generate(eng, [[1, 2, 3]], GenerationOptions(max_tokens=4))[0]) == 4
    word.fill_(1004)
    with pytest.raises(KernelError, match="1004"):
        generate(eng, [[1, 2, 3], [4]], GenerationOptions(max_tokens=4))
    assert eng.cache.slots.n_held == 0


def test_chunked_prompts_give_the_same_tokens(cpu_ops, folders):
    """An engine whose steps are bounded feeds prompts in chunks (mixed with nothing else) and
    sizes the windowed group of Tiny-C by its window; the tokens are those of whole prompts."""
    folder = folders[("C", "float32")]
    prompts = [random_tokens(300, n, 90 + n) for n in (70, 3, 33)]
    whole = generate(cpu_engine(folder), prompts, GenerationOptions(max_tokens=6))
    eng = cpu_engine(folder, max_step_tokens=16, max_sequences=4)
    windowed = [g for g in eng.cache.groups if getattr(g, "spec", None) is not None and getattr(g.spec, "window", None)]
    assert windowed and windowed[0].n_pages == 4 * 2              # window 40 + 15 more tokens: one page, and one more; four slots
    for pipelined in (False, True):
        eng.supports_device_tokens = pipelined
        assert generate(eng, prompts, GenerationOptions(max_tokens=6)) == whole
    with pytest.raises(ValueError, match="at most 16"):
        from wpc_engine_b200 import SequenceStep
        slot = eng.open_sequence()
        try:
            eng.step([SequenceStep(slot, [1] * 17, want=[])])
        finally:
            eng.close_sequence(slot)
    eng.cache.check()


def test_a_draw_with_a_temperature_needs_the_slot_s_own_sampler_state(cpu_ops, folders):
    """A slot keeps the seed and counter of its last occupant; drawing from it before they are
    set anew is refused, so that no request's draws depend on who held the slot before."""
    import torch
    from wpc_engine_b200 import SequenceStep
    eng = cpu_engine(folders[("A", "float32")])
    slot = eng.open_sequence()
    logits = eng.step([SequenceStep(slot, [1, 2, 3], want=[2])])
    assert eng.sample(logits, [slot], 0.0).numel() == 1            # greedy reads no state
    with pytest.raises(ValueError, match="no sampler state"):
        eng.sample(logits, [slot], 0.8)
    eng.set_sampler_state([slot], seed=3, request_ids=[0])
    first = int(eng.sample(logits, [slot], 0.8)[0])
    eng.close_sequence(slot)
    again = eng.open_sequence()
    assert again == slot
    logits = eng.step([SequenceStep(again, [1, 2, 3], want=[2])])
    with pytest.raises(ValueError, match="no sampler state"):
        eng.sample(logits, [again], 0.8)
    eng.set_sampler_state([again], seed=3, request_ids=[0])
    assert int(eng.sample(logits, [again], 0.8)[0]) == first       # the same draw as the first occupant's first
    eng.close_sequence(again)
