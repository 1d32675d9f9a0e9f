"""The generation loop's decisions, with a fake engine: batches in order, stop tokens (kept
in the output, never fed), sequences that end earlier, slots given back and used again."""
import pytest

from wpc_engine_b200.engine.generate import GenerationOptions, _Live, advance, generate, plan_batches
from wpc_engine_b200.sampling import banned_from_env, stop_ids_of_folder, uniform_for


class FakeCache:
    def __init__(self, n_pages, n_slots):
        self.n_pages, self.n_slots = n_pages, n_slots


class FakeEngine:
    """Sequence r answers with r*100 + (number of tokens it has been fed so far)."""

    def __init__(self, n_pages=64, n_slots=4):
        self.cache = FakeCache(n_pages, n_slots)
        self.free = list(range(n_slots))
        self.fed = {}
        self.request_of = {}
        self.log = []
        self.pending = None

    def open_sequence(self):
        s = min(self.free)
        self.free.remove(s)
        self.fed[s] = []
        return s

    def close_sequence(self, s):
        assert s in self.fed
        del self.fed[s]
        self.free.append(s)

    def set_sampler_state(self, slots, seed, requests):
        self.request_of.update(dict(zip(slots, requests)))

    def step(self, entries):
        self.log.append([(e.slot, list(e.tokens), list(e.want)) for e in entries])
        for e in entries:
            self.fed[e.slot].extend(e.tokens)
        self.pending = [e.slot for e in entries]
        return "logits"

    def sample(self, logits, slots, temperature, banned=()):
        assert logits == "logits" and list(slots) == self.pending

        class Ids(list):
            def tolist(self):
                return list(self)
        return Ids(self.request_of[s] * 100 + len(self.fed[s]) for s in slots)


def test_plan_batches_respects_pages_slots_and_order():
    assert plan_batches([10, 10, 10, 10, 10], 20, 64, 4) == [[0, 1, 2, 3], [4]]
    assert plan_batches([100, 100, 100], 28, 4, 8) == [[0, 1], [2]]           # two pages each, four in all
    assert plan_batches([5, 5, 5], 5, 64, 8, max_batch=2) == [[0, 1], [2]]
    with pytest.raises(ValueError, match="empty prompt"):
        plan_batches([3, 0], 5, 64, 8)
    with pytest.raises(ValueError, match="needs 3 pages"):
        plan_batches([130], 10, 2, 8)


def test_advance_stops_on_stop_token_and_on_max_tokens():
    live = [_Live(0, 0), _Live(1, 1, [5]), _Live(2, 2)]
    go_on, done = advance(live, [9, 8, 7], GenerationOptions(max_tokens=2), frozenset([7]))
    assert [s.request for s in go_on] == [0] and [s.request for s in done] == [1, 2]
    assert done[0].output == [5, 8] and done[1].output == [7]        # the stop token stays in the output


def test_loop_feeds_prompts_once_then_one_token_each_and_shrinks_the_batch():
    eng = FakeEngine()
    prompts = [[1, 2, 3], [4], [5, 6]]
    # request 1 answers 101, 102, ...: make 102 a stop token so that it ends after two tokens
    out = generate(eng, prompts, GenerationOptions(max_tokens=4, stop_token_ids=[102]))
    assert out == [[3, 4, 5, 6], [101, 102], [202, 203, 204, 205]]
    assert eng.log[0] == [(0, [1, 2, 3], [2]), (1, [4], [0]), (2, [5, 6], [1])]
    assert eng.log[1] == [(0, [3], [0]), (1, [101], [0]), (2, [202], [0])]
    assert eng.log[2] == [(0, [4], [0]), (2, [203], [0])]             # request 1 left; 102 was never fed
    assert len(eng.log) == 4                                            # no step after the last token
    assert sorted(eng.free) == [0, 1, 2, 3] and not eng.fed


def test_batches_follow_one_another_and_reuse_slots():
    eng = FakeEngine(n_slots=2)
    out = generate(eng, [[1], [2], [3], [4], [5]], GenerationOptions(max_tokens=2))
    assert out == [[1, 2], [101, 102], [201, 202], [301, 302], [401, 402]]
    # per batch: one prompt step, one single-token step; each batch takes the slots that the last gave back
    assert [[e[0] for e in step] for step in eng.log] == [[0, 1], [0, 1], [0, 1], [0, 1], [0], [0]]
    assert [step[0][1] for step in eng.log] == [[1], [1], [3], [201], [5], [401]]
    assert sorted(eng.free) == [0, 1]


def test_slots_come_back_after_an_error():
    eng = FakeEngine()
    eng.sample = lambda *a, **k: (_ for _ in ()).throw(RuntimeError("boom"))
    with pytest.raises(RuntimeError, match="boom"):
        generate(eng, [[1, 2], [3]], GenerationOptions(max_tokens=3))
    assert sorted(eng.free) == [0, 1, 2, 3]


def test_zero_tokens_and_stats():
    eng = FakeEngine()
    assert generate(eng, [[1]], GenerationOptions(max_tokens=0)) == [[]]
    stats = {}
    generate(eng, [[1, 2, 3], [4]], GenerationOptions(max_tokens=3), stats=stats)
    assert stats["prefill_tokens"] == 4 and stats["decode_tokens"] == 4 and stats["decode_steps"] == 2


def test_stop_ids_and_banned_ids_sources(tmp_path, monkeypatch):
    # wpc-runtime/src/main.rs:449-488 and sampling.rs:23-31
    (tmp_path / "generation_config.json").write_text('{"eos_token_id": [9, 3]}')
    (tmp_path / "config.json").write_text('{"eos_token_id": 3}')
    assert stop_ids_of_folder(str(tmp_path)) == [3, 9]
    assert stop_ids_of_folder(str(tmp_path / "none")) == []
    monkeypatch.setenv("WPC_BAN_TOKENS", "1, 2,x,30")
    assert banned_from_env() == [1, 2, 30]
    monkeypatch.delenv("WPC_BAN_TOKENS")
    assert banned_from_env() == []
    assert uniform_for(1, 2, 3) == uniform_for(1, 2, 3) != uniform_for(1, 2, 4)


def test_plan_batches_takes_what_the_cache_says_fits():
    # a model without keys and values: only the slots limit a batch
    assert plan_batches([10 ** 6, 10 ** 6, 5], 10 ** 6, None, 2) == [[0, 1], [2]]
    # the cache's own answer (every group with its own pool)
    seen = []

    def fits(lens):
        seen.append(list(lens))
        return sum(lens) <= 100
    assert plan_batches([30, 30, 30, 30], 10, fits, 8) == [[0, 1], [2, 3]]
    assert [40] in seen and [40, 40, 40] in seen
    with pytest.raises(ValueError, match="request 1 needs"):
        plan_batches([5, 200], 10, fits, 8)


def test_prompts_come_in_chunks_when_steps_are_bounded():
    from wpc_engine_b200.engine.generate import prompt_steps
    steps = prompt_steps([7, 8, 9], [[1, 2, 3, 4, 5], [6], [7, 8, 9]], 2)
    assert [[(e.slot, list(e.tokens), list(e.want)) for e in s] for s in steps] == [
        [(7, [1, 2], []), (8, [6], [0]), (9, [7, 8], [])],
        [(7, [3, 4], []), (9, [9], [0])],
        [(7, [5], [0])]]
    assert len(prompt_steps([1], [[1, 2, 3]], None)) == 1


class ChunkedFake(FakeEngine):
    """Answers with real tensors, so that the loop can put the rows of several prompt steps together."""
    max_step_tokens = 2

    def step(self, entries):
        import torch
        super().step(entries)
        return torch.tensor([[float(self.request_of[e.slot] * 100 + len(self.fed[e.slot]))] for e in entries if len(e.want)])

    def sample(self, logits, slots, temperature, banned=()):
        assert logits.shape[0] == len(slots)
        return logits[:, 0].to(int)


def test_loop_with_bounded_steps_feeds_chunks_then_one_token_each():
    eng = ChunkedFake()
    out = generate(eng, [[1, 2, 3, 4, 5], [6], [7, 8, 9]], GenerationOptions(max_tokens=3))
    assert out == [[5, 6, 7], [101, 102, 103], [203, 204, 205]]
    assert [[len(e[1]) for e in s] for s in eng.log[:3]] == [[2, 1, 2], [2, 1], [1]]
    assert eng.log[3] == [(0, [5], [0]), (1, [101], [0]), (2, [203], [0])]
    assert sorted(eng.free) == [0, 1, 2, 3]
