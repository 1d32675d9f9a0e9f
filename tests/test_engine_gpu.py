"""The engine on the GPU against the plain implementation, in 32-bit and in bfloat16: each
request alone and whole, with its last 32 tokens one by one, and in batches of unequal
lengths whose shorter requests end earlier, one batch after another so that slots and pages
are used again."""
import numpy as np
import pytest
import torch

from helpers import (assert_close_to_plain, bfloat16_bound, random_tokens, run_batch, run_tail_one_by_one, run_whole)
from plain import qwen2_plain as P
from wpc_engine_b200 import Engine, GenerationOptions, generate

pytestmark = pytest.mark.gpu
CASES = [(n, d) for n in ("A", "B", "C") for d in ("float32", "bfloat16")]


@pytest.fixture(scope="module")
def engines(folders):
    made = {}

    def get(name, dtype, **kw):
        key = (name, dtype, tuple(sorted(kw.items())))
        if key not in made:
            made[key] = (Engine.from_folder(folders[(name, dtype)], dtype=dtype, max_tokens=4096, **kw),
                         folders[(name, dtype)])
        return made[key]
    return get


def requests_for(engine, lens, seed=100):
    return [random_tokens(engine.config.vocab_size, n, seed + i) for i, n in enumerate(lens)]


@pytest.mark.parametrize("name,dtype", CASES)
def test_whole(engines, name, dtype):
    eng, folder = engines(name, dtype)
    for r in requests_for(eng, [1, 2, 63, 64, 65, 120]):
        assert_close_to_plain(run_whole(eng, r), folder, r, dtype, f"whole, {len(r)} tokens")


@pytest.mark.parametrize("name,dtype", CASES)
def test_last_32_one_by_one(engines, name, dtype):
    eng, folder = engines(name, dtype)
    for r in requests_for(eng, [5, 33, 100, 127], seed=200):
        assert_close_to_plain(run_tail_one_by_one(eng, r), folder, r, dtype, f"tail, {len(r)} tokens")


@pytest.mark.parametrize("name,dtype", CASES)
def test_unequal_batches_reuse_slots(engines, name, dtype):
    eng, folder = engines(name, dtype)
    for round_, (lens, prompts) in enumerate([([70, 5, 33, 100], [20, 5, 1, 64]),
                                              ([9, 128, 64], [9, 100, 3]),
                                              ([100, 100, 31, 2, 77], [64, 65, 30, 1, 77])]):
        reqs = requests_for(eng, lens, seed=300 + 10 * round_)
        outs = run_batch(eng, reqs, prompts)
        for r, o in zip(reqs, outs):
            assert_close_to_plain(o, folder, r, dtype, f"batch {round_}, {len(r)} tokens")
        eng.cache.check()
        assert eng.cache.slots.n_held == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_chunking_and_batching_change_only_rounding(engines, dtype):
    """The same request whole, tail by tail and inside a batch: the three differ from one
    another far less than the type's distance from the plain implementation."""
    eng, _ = engines("C", dtype)
    r = requests_for(eng, [120], seed=400)[0]
    whole = run_whole(eng, r)
    tail = run_tail_one_by_one(eng, r)
    batch = run_batch(eng, [r, r[:50], r[:7]], [60, 50, 7])[0]
    tol = 2e-5 if dtype == "float32" else 6e-2
    scale = np.abs(whole).max()
    assert np.abs(tail - whole).max() <= tol * scale
    assert np.abs(batch - whole).max() <= tol * scale


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(engines, folders, dtype):
    """300 tokens decoded one by one after a short prompt (graphs replayed, pages crossed)."""
    eng, folder = engines("C", dtype)
    r = requests_for(eng, [330], seed=500)[0]
    got = run_tail_one_by_one(eng, r, tail=300)
    assert_close_to_plain(got, folder, r, dtype, "long decoding")


def test_greedy_generation_matches_plain(engines):
    eng, folder = engines("A", "float32")
    cfg, tensors = P.read_model_folder(folder)
    prompts = [random_tokens(256, n, 40 + n) for n in (5, 11, 17)]
    got = generate(eng, prompts, GenerationOptions(max_tokens=8))
    for p, g in zip(prompts, got):
        assert g == P.generate_greedy(cfg, tensors, p, 8)
    eng.cache.check()


@pytest.mark.parametrize("name,dtype", CASES)
def test_first_tokens_of_a_sequence(engines, name, dtype):
    """Position 0, the first decoded token after a one-token prompt, and a prompt's end."""
    eng, folder = engines(name, dtype)
    r = requests_for(eng, [6], seed=700)[0]
    slot = eng.open_sequence()
    try:
        from wpc_engine_b200 import SequenceStep
        rows = [eng.step([SequenceStep(slot, [t], want=[0])]).float().cpu().numpy() for t in r]
    finally:
        eng.close_sequence(slot)
    assert_close_to_plain(np.concatenate(rows), folder, r, dtype, "one token at a time from the start")


def test_temperature_generation_follows_the_plain_sampler(engines):
    """Tiny-B, temperature 0.8, seed 7: every drawn token is what the plain sampler draws from
    the engine's own logits with the same uniform number; batching changes no draw."""
    eng, folder = engines("B", "float32")
    prompts = [random_tokens(384, n, 50 + n) for n in (1, 7, 23, 40)]
    opts = GenerationOptions(max_tokens=12, temperature=0.8, seed=7)
    got = generate(eng, prompts, opts)
    assert [len(g) for g in got] == [12] * 4
    for r, (p, g) in enumerate(zip(prompts, got)):
        logits = run_whole(eng, p + g[:-1])[len(p) - 1:]
        for step, tok in enumerate(g):
            u = P.uniform_for(7, r, step)
            idx, cdf, target = P.sample_temperature(logits[step], 0.8, u)
            lo = cdf[tok - 1] if tok > 0 else 0.0
            slack = 1e-4 * cdf[-1]
            assert lo - slack <= target <= cdf[tok] + slack, (r, step, tok, idx)
    alone = generate(eng, [prompts[2]], opts)
    # request numbers are positions in the call, so the same prompt alone is request 0: other draws
    again = generate(eng, prompts, opts)
    assert again == got and len(alone[0]) == 12


def test_stop_tokens_end_one_sequence_while_others_go_on(engines):
    eng, folder = engines("A", "float32")
    prompts = [random_tokens(256, n, 40 + n) for n in (5, 11, 17)]
    free = generate(eng, prompts, GenerationOptions(max_tokens=8))
    stop = free[1][2]
    got = generate(eng, prompts, GenerationOptions(max_tokens=8, stop_token_ids=[stop]))
    for f, g in zip(free, got):
        cut = f.index(stop) + 1 if stop in f else len(f)
        assert g == f[:cut]
    eng.cache.check()
    assert eng.cache.slots.n_held == 0


ODD = {
    # head size over 128 (plain attention), width 8 does not divide (plain products), odd vocabulary
    "wide_head": dict(num_hidden_layers=2, hidden_size=100, num_attention_heads=2, num_key_value_heads=1, head_dim=144,
                      intermediate_size=52, vocab_size=333, rope_theta=7000.0, rms_norm_eps=2e-6),
    # 32 query heads on one KV head (more than the tensor-core kernel stacks), tied head
    "many_per_group": dict(num_hidden_layers=1, hidden_size=512, num_attention_heads=32, num_key_value_heads=1,
                           intermediate_size=192, vocab_size=200, rope_theta=1e5, rms_norm_eps=1e-5,
                           tie_word_embeddings=True),
    # many heads and groups that are no power of two, head size 80, window on every layer
    "odd_heads": dict(num_hidden_layers=2, hidden_size=240, num_attention_heads=6, num_key_value_heads=3, head_dim=80,
                      intermediate_size=320, vocab_size=1000, rope_theta=1e4, rms_norm_eps=1e-6,
                      use_sliding_window=True, sliding_window=70, max_window_layers=0),
}


@pytest.mark.parametrize("name", sorted(ODD))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unusual_sizes(tmp_path_factory, name, dtype):
    """Sizes that the fast kernels do not take run on the plain kernels of the library, and
    sizes that they do take at their edges, with the same answers."""
    from conftest import make_folder
    raw = dict(architectures=["Qwen2ForCausalLM"], tie_word_embeddings=False, max_position_embeddings=512)
    raw.update(ODD[name])
    folder = make_folder(tmp_path_factory, raw, 9, getattr(torch, dtype))
    eng = Engine.from_folder(folder, dtype=dtype, max_tokens=2048)
    reqs = [random_tokens(raw["vocab_size"], n, 800 + n) for n in (150, 9)]
    assert_close_to_plain(run_whole(eng, reqs[0]), folder, reqs[0], dtype, f"{name} whole")
    assert_close_to_plain(run_tail_one_by_one(eng, reqs[0], tail=40), folder, reqs[0], dtype, f"{name} tail")
    for r, o in zip(reqs, run_batch(eng, reqs, [100, 9])):
        assert_close_to_plain(o, folder, r, dtype, f"{name} batch")
    eng.cache.check()


def test_errors_are_loud(engines):
    from wpc_engine_b200 import CacheError, SequenceStep
    eng, _ = engines("A", "float32")
    slot = eng.open_sequence()
    try:
        with pytest.raises(ValueError, match="token id outside"):
            eng.step([SequenceStep(slot, [256], want=[0])])
        with pytest.raises(ValueError, match="longest sequence"):
            eng.step([SequenceStep(slot, [1] * 129, want=[0])])
        with pytest.raises(ValueError, match="twice"):
            eng.step([SequenceStep(slot, [1], want=[0]), SequenceStep(slot, [2], want=[0])])
        with pytest.raises(CacheError, match="not open"):
            eng.step([SequenceStep(slot + 1000, [1], want=[0])])
        assert eng.sequence_length(slot) == 0
    finally:
        eng.close_sequence(slot)
    small = Engine.from_folder(engines("A", "float32")[1], dtype="float32", max_tokens=128)
    a, b, c = small.open_sequence(), small.open_sequence(), None
    small.step([SequenceStep(a, [1] * 64, want=[]), SequenceStep(b, [2] * 64, want=[])])
    with pytest.raises(CacheError, match="out of pages"):
        small.step([SequenceStep(a, [3], want=[0])])
    with pytest.raises(CacheError, match="out of slots"):
        small.open_sequence()
    small.close_sequence(a)
    assert small.step([SequenceStep(b, [3], want=[0])]).shape == (1, 256)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_prompt_in_chunks(tmp_path_factory, dtype):
    """A 5,000-token request fed in chunks of 1,024 and then one token at a time, beside a
    short request: many pages, chunks that attend to a deep cache, long decode contexts."""
    from conftest import make_folder
    from wpc_engine_b200 import SequenceStep
    raw = dict(architectures=["Qwen2ForCausalLM"], num_hidden_layers=2, hidden_size=128, num_attention_heads=2,
               num_key_value_heads=1, intermediate_size=192, vocab_size=500, rope_theta=1e6, rms_norm_eps=1e-6,
               max_position_embeddings=8192, tie_word_embeddings=True)
    folder = make_folder(tmp_path_factory, raw, 21, getattr(torch, dtype))
    eng = Engine.from_folder(folder, dtype=dtype, max_tokens=8192)
    long_req, short_req = random_tokens(500, 5008, 900), random_tokens(500, 40, 901)
    want = P.forward(*P.read_model_folder(folder), long_req, np.float64)
    a, b = eng.open_sequence(), eng.open_sequence()
    rows = []
    try:
        fed = 0
        while fed < 5000:
            n = min(1024, 5000 - fed)
            entries = [SequenceStep(a, long_req[fed:fed + n], want=[n - 1])]
            if fed == 0:
                entries.append(SequenceStep(b, short_req, want=[]))
            rows.append((fed + n - 1, eng.step(entries).float().cpu().numpy()[0]))
            fed += n
        for i in range(5000, 5008):
            out = eng.step([SequenceStep(a, [long_req[i]], want=[0]), SequenceStep(b, [short_req[i % 40]], want=[0])])
            rows.append((i, out.float().cpu().numpy()[0]))
    finally:
        eng.close_sequence(a)
        eng.close_sequence(b)
    bound = 4 * np.abs(P.forward(*P.read_model_folder(folder), long_req[:600], np.float32)
                       - want[:600]).max() + 1e-5 if dtype == "float32" else bfloat16_bound(want)
    for place, got in rows:
        err = np.abs(got - want[place]).max()
        assert err <= bound, (place, err, bound)
    eng.cache.check()


def test_one_long_sequence_decodes_with_several_clusters_to_a_pair(tmp_path_factory):
    """At 12,000 positions a single sequence's decode attention is planned with several clusters
    to each (sequence, kv head) pair, whose parts a ticket's last cluster adds.  The same positions
    are reached once by single-token steps (replayed from a graph) and once inside a prompt's
    last chunk, where the prefill kernels serve them; both must agree within bfloat16's noise,
    and both with the float32 path."""
    from conftest import make_folder
    from wpc_engine_b200 import SequenceStep, ops
    raw = dict(architectures=["Qwen2ForCausalLM"], num_hidden_layers=2, hidden_size=128, num_attention_heads=2,
               num_key_value_heads=1, intermediate_size=192, vocab_size=500, rope_theta=1e6, rms_norm_eps=1e-6,
               max_position_embeddings=16384, tie_word_embeddings=True)
    folder = make_folder(tmp_path_factory, raw, 22, torch.bfloat16)
    n, tail = 12000, 4
    cluster, groups = ops.plan_decode_cluster(1, 1, 2, 64, n + tail, None)
    assert cluster >= 2 and groups > 1, (cluster, groups)
    tokens = random_tokens(500, n + tail, 902)

    def chunks(eng, slot, upto, want_from):
        rows, fed = [], 0
        while fed < upto:
            m = min(2048, upto - fed)
            want = [i - fed for i in range(max(fed, want_from), fed + m)]
            out = eng.step([SequenceStep(slot, tokens[fed:fed + m], want=want)])
            rows += list(out.float().cpu().numpy()) if want else []
            fed += m
        return rows

    got = {}
    for dtype in ("bfloat16", "float32"):
        eng = Engine.from_folder(folder, dtype=dtype, max_tokens=2 * 12288 + 128)
        a, b = eng.open_sequence(), eng.open_sequence()
        try:
            chunks(eng, a, n, n)
            one_by_one = [eng.step([SequenceStep(a, [tokens[i]], want=[0])]).float().cpu().numpy()[0]
                          for i in range(n, n + tail)]
            in_prompt = chunks(eng, b, n + tail, n)
        finally:
            eng.close_sequence(a)
            eng.close_sequence(b)
        eng.cache.check()
        got[dtype] = (np.stack(one_by_one), np.stack(in_prompt))
        assert ops.device_status() == 0
    exact = got["float32"][1]
    bound = bfloat16_bound(exact)
    assert np.abs(got["float32"][0] - exact).max() <= 1e-3 * np.abs(exact).max()
    for rows in got["bfloat16"]:
        assert np.abs(rows - exact).max() <= bound, (np.abs(rows - exact).max(), bound)


def test_medium_model_graphs_and_dependent_launch_change_nothing(tmp_path_factory):
    """A model large enough for the real tile shapes (split-K products, weight tiles fetched
    ahead, many CTAs per attention pair, persistent prefill products, tcgen05 attention):
    single-token steps replayed from graphs with programmatic dependent launch against the same
    steps launched one by one without it, and both against the float32 path."""
    from conftest import make_folder
    from wpc_engine_b200 import SequenceStep, ops
    raw = dict(architectures=["Qwen2ForCausalLM"], num_hidden_layers=3, hidden_size=1024, num_attention_heads=8,
               num_key_value_heads=2, intermediate_size=2816, vocab_size=3000, rope_theta=1e6, rms_norm_eps=1e-6,
               max_position_embeddings=4096, tie_word_embeddings=False, use_sliding_window=True,
               sliding_window=200, max_window_layers=1)
    folder = make_folder(tmp_path_factory, raw, 31, torch.bfloat16)
    reqs = [random_tokens(3000, n, 970 + n) for n in (700, 130, 9, 333)]

    def run(dtype, graphs, pdl):
        was = ops.set_pdl(pdl)
        try:
            eng = Engine.from_folder(folder, dtype=dtype, max_tokens=8192, use_graphs=graphs)
            slots = [eng.open_sequence() for _ in reqs]
            out = [eng.step([SequenceStep(s, r, want=[len(r) - 1]) for s, r in zip(slots, reqs)]).float().cpu().numpy()]
            for i in range(70):          # crosses page boundaries; the first step of a shape runs directly
                toks = [int(r[(i * 7) % len(r)]) for r in reqs]
                out.append(eng.step([SequenceStep(s, [t], want=[0]) for s, t in zip(slots, toks)]).float().cpu().numpy())
            for s in slots:
                eng.close_sequence(s)
            eng.cache.check()
            assert ops.device_status() == 0
            return np.stack(out)
        finally:
            ops.set_pdl(was)

    fast = run("bfloat16", True, True)
    slow = run("bfloat16", False, False)
    full = run("float32", False, False)
    scale = np.abs(full).max()
    # the same kernels either way: only the order of the red.add shares may differ
    assert np.abs(fast - slow).max() <= 2e-2 * scale
    assert np.abs(fast - full).max() <= 6e-2 * scale and np.abs(slow - full).max() <= 6e-2 * scale


def test_medium_model_long_prompt_whole_and_in_chunks(tmp_path_factory):
    """A prompt long enough for the many-token kernels (256-row tiles on pairs of SMs, the
    q/k/v product that rotates and writes the cache in its epilogue, tcgen05 attention with
    a window): whole, in two chunks, and with its tail token by token, in bfloat16 against
    the float32 path."""
    from conftest import make_folder
    from wpc_engine_b200 import SequenceStep, ops
    raw = dict(architectures=["Qwen2ForCausalLM"], num_hidden_layers=2, hidden_size=1024, num_attention_heads=8,
               num_key_value_heads=2, intermediate_size=2816, vocab_size=3000, rope_theta=1e6, rms_norm_eps=1e-6,
               max_position_embeddings=4096, tie_word_embeddings=False, use_sliding_window=True,
               sliding_window=300, max_window_layers=1)
    folder = make_folder(tmp_path_factory, raw, 37, torch.bfloat16)
    req = random_tokens(3000, 2100, 4242)
    want = [0, 5, 1023, 1024, 1791, 1792, 2047, 2099]

    def run(dtype, cuts):
        eng = Engine.from_folder(folder, dtype=dtype, max_tokens=4096)
        slot = eng.open_sequence()
        rows = []
        for lo, hi in zip(cuts[:-1], cuts[1:]):
            w = [p - lo for p in want if lo <= p < hi]
            out = eng.step([SequenceStep(slot, req[lo:hi], want=w)])
            if w:
                rows.append(out.float().cpu().numpy())
        eng.close_sequence(slot)
        eng.cache.check()
        assert ops.device_status() == 0
        return np.concatenate(rows)

    whole = run("bfloat16", [0, 2100])
    halves = run("bfloat16", [0, 1792, 2100])
    tail = run("bfloat16", [0, 2090] + list(range(2091, 2101)))
    full = run("float32", [0, 2100])
    scale = np.abs(full).max()
    assert np.abs(whole - full).max() <= 6e-2 * scale
    assert np.abs(halves - full).max() <= 6e-2 * scale
    assert np.abs(tail - full).max() <= 6e-2 * scale
    assert np.abs(whole - halves).max() <= 3e-2 * scale and np.abs(whole - tail).max() <= 3e-2 * scale
