"""Schedules of the step function beyond "all prompts, then one token each", against the plain
implementation: steps that mix sequences bringing one token with sequences bringing many, a
model with 128-wide heads and seven query heads to a KV head, two layers of the
Qwen2.5-7B shape, and single-token steps of more sequences than the device has SMs."""
import numpy as np
import pytest
import torch

from conftest import make_folder
from helpers import assert_close_to_plain, bfloat16_bound, random_tokens, run_batch, run_tail_one_by_one, run_whole
from plain import qwen2_plain as P
from wpc_engine_b200 import Engine, SequenceStep

pytestmark = pytest.mark.gpu
CASES = [(n, d) for n in ("A", "B", "C") for d in ("float32", "bfloat16")]


def run_schedule(engine, requests, schedule):
    """schedule: a list of steps, each a list of (request number, tokens it brings now).  A
    request's slot is opened at its first step and closed after the step that brings its last
    token.  Every fed place is wanted; returns the logits of every request: list of [T_i, V]."""
    slots, fed = {}, [0] * len(requests)
    rows = [[] for _ in requests]
    try:
        for step in schedule:
            entries = []
            for r, n in step:
                if r not in slots:
                    slots[r] = engine.open_sequence()
                entries.append(SequenceStep(slots[r], requests[r][fed[r]: fed[r] + n], want=list(range(n))))
            out = engine.step(entries).float().cpu().numpy()
            at = 0
            for r, n in step:
                rows[r].append(out[at: at + n])
                at += n
                fed[r] += n
                if fed[r] == len(requests[r]):
                    engine.close_sequence(slots.pop(r))
    finally:
        for s in slots.values():
            engine.close_sequence(s)
    assert fed == [len(r) for r in requests]
    return [np.concatenate(r, axis=0) for r in rows]


@pytest.mark.parametrize("name,dtype", CASES)
def test_steps_that_mix_one_token_and_many(folders, name, dtype):
    """Request 0 brings its prompt; from then on it decodes one token a step while request 1
    arrives in chunks of 40, 17 and 1 and request 2 starts with a one-token prompt; later a
    fourth request joins with a whole prompt while the others decode; each ends at its own time."""
    folder = folders[(name, dtype)]
    eng = Engine.from_folder(folder, dtype=dtype, max_tokens=2048)
    reqs = [random_tokens(eng.config.vocab_size, n, 1200 + n) for n in (78, 64, 8, 38)]
    schedule = [[(0, 70)],
                [(0, 1), (1, 40), (2, 1)],
                [(0, 1), (1, 17), (2, 1)],
                [(0, 1), (1, 1), (2, 1)],
                [(0, 1), (1, 1), (2, 1), (3, 30)],
                [(0, 1), (1, 1), (2, 1), (3, 1)],
                [(0, 1), (1, 1), (2, 1), (3, 1)],
                [(0, 1), (1, 1), (2, 1), (3, 1)],
                [(0, 1), (1, 1), (2, 1), (3, 4)],        # request 0 and 2 end here
                [(1, 1), (3, 1)],                        # request 3 ends, request 1 ends
                ]
    outs = run_schedule(eng, reqs, schedule)
    for i, (r, o) in enumerate(zip(reqs, outs)):
        assert_close_to_plain(o, folder, r, dtype, f"{name} mixed steps, request {i}")
    eng.cache.check()
    assert eng.cache.slots.n_held == 0


@pytest.mark.parametrize("name,dtype", CASES)
@pytest.mark.parametrize("seed", [11, 12, 13])
def test_random_schedules(folders, name, dtype, seed):
    """Schedules drawn at random (a fixed seed each): requests join while others run, steps bring
    one token each or chunks of any size or a mixture, only some places are wanted, the pool of
    pages is small enough to run out (the step that asked for too much leaves the cache as it
    was, and the longest request is closed to make room), slots and pages come back and are used
    again.  Every wanted row against the plain implementation."""
    from wpc_engine_b200 import CacheError
    rng = np.random.default_rng(seed)
    folder = folders[(name, dtype)]
    eng = Engine.from_folder(folder, dtype=dtype, max_tokens=int(rng.choice([320, 512, 1024])), max_sequences=5)
    cfg, tensors = P.read_model_folder(folder)
    longest = min(600, eng.config.max_position_embeddings)
    reqs = [random_tokens(eng.config.vocab_size, int(rng.integers(1, longest + 1)), 7000 + 10 * seed + i) for i in range(7)]
    plain, fed, slots, waiting = {}, [0] * len(reqs), {}, list(range(len(reqs)))
    bound = None
    compared = evicted = 0
    try:
        for _ in range(4000):
            if not (waiting or slots):
                break
            while waiting and len(slots) < 5 and rng.random() < 0.5:
                slots[waiting.pop(0)] = eng.open_sequence()
            if not slots:
                continue
            active = [r for r in slots if rng.random() < 0.8] or list(slots)[:1]
            single = rng.random() < 0.7
            entries, brought = [], []
            for r in active:
                left = len(reqs[r]) - fed[r]
                n = 1 if single else max(1, min(left, int(rng.choice([1, 1, 2, 7, 40, 64, 65, 130, 300]))))
                want = (sorted({int(x) for x in rng.integers(0, n, size=int(rng.integers(0, 4)))})
                        if rng.random() < 0.7 else list(range(n)))
                entries.append(SequenceStep(slots[r], reqs[r][fed[r]: fed[r] + n], want=want))
                brought.append((r, n, want))
            try:
                out = eng.step(entries)
            except CacheError:
                eng.cache.check()
                r = max(slots, key=lambda r: fed[r])
                eng.close_sequence(slots.pop(r))
                evicted += 1
                continue
            out = None if out is None else out.float().cpu().numpy()     # nothing wanted: nothing returned
            at = 0
            for r, n, want in brought:
                if want:
                    if r not in plain:
                        plain[r] = P.forward(cfg, tensors, reqs[r], np.float64)
                    ref = plain[r][[fed[r] + i for i in want]]
                    bound = bfloat16_bound(plain[r]) if dtype == "bfloat16" else 1e-3 * np.abs(plain[r]).max()
                    err = np.abs(out[at: at + len(want)] - ref).max()
                    assert err <= bound, (seed, r, fed[r], n, want, err, bound, [(b[0], b[1]) for b in brought])
                    at += len(want)
                    compared += len(want)
                fed[r] += n
                if fed[r] >= len(reqs[r]):
                    eng.close_sequence(slots.pop(r))
    finally:
        for s_ in slots.values():
            eng.close_sequence(s_)
    assert compared > 50
    eng.cache.check()
    assert eng.cache.slots.n_held == 0


WIDE_GROUP = dict(architectures=["Qwen2ForCausalLM"], num_hidden_layers=2, hidden_size=896, num_attention_heads=7,
                  num_key_value_heads=1, head_dim=128, intermediate_size=1536, vocab_size=1000, rope_theta=1e6,
                  rms_norm_eps=1e-6, max_position_embeddings=2048, tie_word_embeddings=False)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_heads_of_128_seven_to_a_group(tmp_path_factory, dtype):
    """head_dim 128 with seven query heads to one KV head (the grouping of the 7B shape), in a
    model small enough for the plain implementation: whole, tail one by one, unequal batches."""
    folder = make_folder(tmp_path_factory, WIDE_GROUP, 51, getattr(torch, dtype))
    eng = Engine.from_folder(folder, dtype=dtype, max_tokens=4096)
    reqs = [random_tokens(1000, n, 1300 + n) for n in (300, 70, 33)]
    assert_close_to_plain(run_whole(eng, reqs[0]), folder, reqs[0], dtype, "whole")
    assert_close_to_plain(run_tail_one_by_one(eng, reqs[0]), folder, reqs[0], dtype, "tail")
    for round_ in range(2):                 # the second batch takes the slots and pages of the first
        for r, o in zip(reqs, run_batch(eng, reqs, [260, 64, 1])):
            assert_close_to_plain(o, folder, r, dtype, f"batch {round_}")
    eng.cache.check()
    assert eng.cache.slots.n_held == 0


@pytest.fixture(scope="module")
def real_shape(tmp_path_factory):
    """Two layers of the Qwen2.5-7B shape as a folder, and the plain implementation's float64
    logits of three requests at a few dozen places each (the layers run on whole requests; the
    output head, 152,064 rows, only at the compared places)."""
    raw = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", num_hidden_layers=2, hidden_size=3584,
               num_attention_heads=28, num_key_value_heads=4, intermediate_size=18944, vocab_size=152064,
               rope_theta=1000000.0, rms_norm_eps=1e-6, max_position_embeddings=32768, tie_word_embeddings=False)
    folder = make_folder(tmp_path_factory, raw, 61, torch.bfloat16)
    cfg, tensors = P.read_model_folder(folder)
    rng = np.random.default_rng(5)
    reqs = [rng.integers(0, 152064, size=n).tolist() for n in (300, 41, 130)]
    rows = [sorted(set(range(0, n, 16)) | set(range(max(0, n - 33), n))) for n in (300, 41, 130)]
    want64 = [P.forward(cfg, tensors, r, np.float64, rows=w) for r, w in zip(reqs, rows)]
    # the plain implementation's own float32 rounding, the yardstick of the 32-bit engine
    noise = [np.abs(P.forward(cfg, tensors, r, np.float32, rows=w).astype(np.float64) - w64).max()
             for r, w, w64 in zip(reqs, rows, want64)]
    del tensors
    return folder, reqs, rows, want64, noise


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_real_layer_shape_against_plain(real_shape, dtype):
    """The engine in 32-bit and in bfloat16 on two layers of the 7B shape against the plain
    implementation in float64: a whole prompt, its last 32 tokens one by one, and an unequal
    batch of three whose shorter requests end earlier."""
    folder, reqs, rows, want64, noise = real_shape
    eng = Engine.from_folder(folder, dtype=dtype, max_tokens=2048, max_sequences=4)

    def check(got, i, what):
        err = np.abs(got.astype(np.float64) - want64[i]).max()
        bound = 4 * noise[i] + 1e-6 if dtype == "float32" else bfloat16_bound(want64[i])
        assert err <= bound, f"{what}: max error {err:.3e} exceeds {bound:.3e}"

    def wanted(i, lo, hi):       # places of request i inside tokens lo .. hi - 1, relative to lo
        return [p - lo for p in rows[i] if lo <= p < hi]

    # whole
    slot = eng.open_sequence()
    got = eng.step([SequenceStep(slot, reqs[0], want=rows[0])]).float().cpu().numpy()
    eng.close_sequence(slot)
    check(got, 0, "whole")
    # the last 32 one by one
    n = len(reqs[0])
    slot = eng.open_sequence()
    parts = [eng.step([SequenceStep(slot, reqs[0][: n - 32], want=wanted(0, 0, n - 32))]).float().cpu().numpy()]
    for t in range(n - 32, n):
        out = eng.step([SequenceStep(slot, [reqs[0][t]], want=wanted(0, t, t + 1))])
        if out is not None:
            parts.append(out.float().cpu().numpy())
    eng.close_sequence(slot)
    check(np.concatenate(parts), 0, "tail one by one")
    # an unequal batch: prompts of 260, 9 and 100 tokens, then one token each until each ends
    prompt_lens = [260, 9, 100]
    slots = [eng.open_sequence() for _ in reqs]
    got = [[] for _ in reqs]
    fed = list(prompt_lens)
    live = [0, 1, 2]
    entries = [SequenceStep(slots[i], reqs[i][:fed[i]], want=wanted(i, 0, fed[i])) for i in live]
    while live:
        out = eng.step(entries)
        at = 0
        for i, e in zip(live, entries):
            if len(e.want):
                got[i].append(out[at: at + len(e.want)].float().cpu().numpy())
                at += len(e.want)
        for i in list(live):
            if fed[i] == len(reqs[i]):
                eng.close_sequence(slots[i])
                live.remove(i)
        entries = [SequenceStep(slots[i], [reqs[i][fed[i]]], want=wanted(i, fed[i], fed[i] + 1)) for i in live]
        for i in live:
            fed[i] += 1
    for i in range(3):
        check(np.concatenate(got[i]), i, f"batch, request {i}")
    eng.cache.check()
    assert eng.cache.slots.n_held == 0


MANY = dict(architectures=["Qwen2ForCausalLM"], num_hidden_layers=2, hidden_size=128, num_attention_heads=2,
            num_key_value_heads=1, head_dim=64, intermediate_size=192, vocab_size=400, rope_theta=1e6,
            rms_norm_eps=1e-5, max_position_embeddings=512, tie_word_embeddings=False)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n_seqs", [160, 300, 1100])
def test_more_sequences_than_ctas(tmp_path_factory, dtype, n_seqs):
    """Single-token steps of many sequences of unequal lengths: more (sequence, KV head) pairs
    than the decode grid has CTAs (a CTA then walks several pairs), more tokens than the
    few-token products take (130 and up), and beyond 1,024 sequences the route through the
    prefill attention.  Every sequence's logits against the plain implementation."""
    folder = make_folder(tmp_path_factory, MANY, 71, getattr(torch, dtype))
    cfg, tensors = P.read_model_folder(folder)
    eng = Engine.from_folder(folder, dtype=dtype, max_tokens=n_seqs * 192, max_sequences=n_seqs)
    rng = np.random.default_rng(n_seqs)
    lens = rng.integers(1, 120, size=n_seqs).tolist()
    lens[0], lens[1], lens[2] = 1, 64, 65
    reqs = [rng.integers(0, 400, size=n + 2).tolist() for n in lens]
    slots = [eng.open_sequence() for _ in reqs]
    eng.step([SequenceStep(s, r[:n], want=[]) for s, r, n in zip(slots, reqs, lens)])
    outs = []
    for k in range(2):        # the first step of a shape runs directly, the second from a graph
        out = eng.step([SequenceStep(s, [r[n + k]], want=[0]) for s, r, n in zip(slots, reqs, lens)])
        outs.append(out.float().cpu().numpy())
    for s in slots:
        eng.close_sequence(s)
    eng.cache.check()
    for i in range(0, n_seqs, 7 if n_seqs > 200 else 1):
        want = P.forward(cfg, tensors, reqs[i], np.float64, rows=[lens[i], lens[i] + 1])
        for k in range(2):
            err = np.abs(outs[k][i] - want[k]).max()
            if dtype == "float32":
                noise = np.abs(P.forward(cfg, tensors, reqs[i], np.float32, rows=[lens[i] + k]).astype(np.float64) - want[k]).max()
                bound = 4 * noise + 1e-6
            else:
                bound = bfloat16_bound(want)
            assert err <= bound, (i, k, lens[i], err, bound)


def test_logits_of_a_step_survive_the_next_step(folders):
    """Single-token steps are replayed from CUDA graphs whose output buffer is reused: the
    tensor that `step` hands out must still hold its own step's logits afterwards."""
    eng = Engine.from_folder(folders[("A", "bfloat16")], dtype="bfloat16", max_tokens=512)
    assert eng.use_graphs
    slot = eng.open_sequence()
    eng.step([SequenceStep(slot, [1, 2, 3], want=[])])
    kept, copies = [], []
    for t in (7, 8, 9, 10, 11):
        out = eng.step([SequenceStep(slot, [t], want=[0])])
        kept.append(out)
        copies.append(out.clone())
    borrowed = eng.step([SequenceStep(slot, [12], want=[0])], borrow=True)
    eng.step([SequenceStep(slot, [13], want=[0])], borrow=True)
    eng.close_sequence(slot)
    assert eng.graph_launches > 0
    for k, c in zip(kept, copies):
        assert torch.equal(k, c)
    assert not any(torch.equal(kept[i], kept[i + 1]) for i in range(4))
    assert borrowed.shape == kept[0].shape
