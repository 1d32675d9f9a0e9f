"""The cache's bookkeeping: no slot or page lost, held twice or freed twice; groups with their
own storage; windows give pages back; and the step plan's layout."""
import random

import numpy as np
import pytest
import torch

from wpc_engine_b200.cache import PAGE, CacheError, FreeList, KVGroup, SequenceCache, StateGroup, pages_for
from wpc_engine_b200.engine.batch import SequenceStep, StepLayout, context_from, plan_step
from wpc_engine_b200.parts.base import KVSpec, StateSpec


def test_free_list_refuses_misuse():
    fl = FreeList(3, "page")
    assert [fl.take(), fl.take(), fl.take()] == [0, 1, 2]
    with pytest.raises(CacheError, match="out of pages"):
        fl.take()
    fl.give_back(1)
    with pytest.raises(CacheError, match="not held"):
        fl.give_back(1)
    with pytest.raises(CacheError, match="does not exist"):
        fl.give_back(3)
    assert fl.take() == 1                      # what was freed is used again first
    fl.check()
    with pytest.raises(CacheError, match="2 wanted"):
        FreeList(1, "slot").take_many(2)


def make_cache(max_tokens=64 * 20, window=40):
    specs = [KVSpec(2, 16), KVSpec(2, 16, window), KVSpec(2, 16, window), StateSpec((3, 5)), None, KVSpec(2, 16)]
    return SequenceCache(specs, max_tokens, torch.float32, "cpu", max_sequences=6)


def test_groups_have_storage_of_their_own():
    c = make_cache()
    kinds = [type(g) for g in c.groups]
    assert kinds.count(KVGroup) == 2 and kinds.count(StateGroup) == 1
    full = c.groups[c.layer_group[0]]
    windowed = c.groups[c.layer_group[1]]
    assert c.layer_group[0] == c.layer_group[5] and c.layer_group[1] == c.layer_group[2] != c.layer_group[0]
    assert full.k.shape == (2, 20, 2, PAGE, 16) and windowed.k.shape == (2, 20, 2, PAGE, 16)
    assert full.k.data_ptr() != windowed.k.data_ptr() and full.pool is not windowed.pool
    assert c.groups[c.layer_group[3]].state.shape == (1, 6, 3, 5) and c.layer_group[4] is None
    assert c.seq_state.shape == (6, 4)


def test_slots_and_pages_are_given_back_and_used_again():
    c = make_cache()
    a, b = c.open(), c.open()
    assert (a, b) == (0, 1)
    assert c.reserve(a, 100) == 0
    c.commit(a, 100)
    assert c.reserve(a, 1) == 100 and c.length(a) == 100
    c.commit(a, 1)
    c.reserve(b, 5)
    c.commit(b, 5)
    full = c.groups[c.layer_group[0]]
    assert len(full.tables[a]) == 2 and len(full.tables[b]) == 1 and full.pool.n_held == 3
    c.check()
    c.close(a)
    with pytest.raises(CacheError, match="not open"):
        c.close(a)
    assert c.open() == 0                        # the slot is used again
    assert full.pool.n_held == 1
    c.check()


def test_window_group_gives_back_pages_that_no_query_can_see():
    c = make_cache(window=40)
    s = c.open()
    windowed = c.groups[c.layer_group[1]]
    full = c.groups[c.layer_group[0]]
    for _ in range(10):
        c.reserve(s, 50)
        c.commit(s, 50)
    # 500 positions; the next query (at 500) sees 461..500: blocks 0..6 are gone
    assert windowed.tables[s][:7] == [-1] * 7 and all(p >= 0 for p in windowed.tables[s][7:])
    assert windowed.pool.n_held == 1 and full.pool.n_held == pages_for(500)
    c.check()
    c.close(s)
    assert windowed.pool.n_held == 0 and full.pool.n_held == 0


def test_exhaustion_is_an_error_not_a_wrong_result():
    c = SequenceCache([KVSpec(1, 8)], 64 * 3, torch.float32, "cpu")
    a, b = c.open(), c.open()
    c.reserve(a, 128)
    c.commit(a, 128)
    with pytest.raises(CacheError, match="out of pages"):
        c.reserve(b, 65)
    c.close(a)
    c.reserve(b, 65)
    c.check()


def test_random_traffic_never_loses_or_doubles_anything():
    rng = random.Random(0)
    c = make_cache(max_tokens=64 * 40)
    live = {}
    for _ in range(400):
        if live and (rng.random() < 0.3 or len(live) == 6):
            s = rng.choice(list(live))
            c.close(s)
            del live[s]
        elif rng.random() < 0.4 and len(live) < 6:
            live[c.open()] = 0
        elif live:
            s = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 7, 64, 65])
            if live[s] + n <= 300:
                c.reserve(s, n)
                c.commit(s, n)
                live[s] += n
        c.check()
        assert set(c.lengths) == set(live) and all(c.length(s) == n for s, n in live.items())
    for s in list(live):
        c.close(s)
    c.check()
    assert c.slots.n_held == 0 and all(g.pool.n_held == 0 for g in c.groups if isinstance(g, KVGroup))


def test_step_plan_layout():
    entries = [SequenceStep(4, [10, 11, 12], want=[0, 2]), SequenceStep(2, [20], want=[]), SequenceStep(7, [30, 31], want=[1])]
    rows = [[[5, 6, -1, -1], [1, -1, -1, -1], [0, 2, 3, -1]]]
    plan = plan_step(entries, [64, 0, 130], rows, 4)
    ctx = context_from(torch.from_numpy(plan.host), plan.layout, torch.float32, plan.max_new_tokens,
                       plan.max_ctx_len, plan.is_decode)
    assert ctx.tokens.tolist() == [10, 11, 12, 20, 30, 31]
    assert ctx.positions.tolist() == [64, 65, 66, 0, 130, 131]
    assert ctx.seq_of_token.tolist() == [0, 0, 0, 1, 2, 2]
    assert ctx.cu_seqlens.tolist() == [0, 3, 4, 6] and ctx.ctx_lens.tolist() == [67, 1, 132]
    assert ctx.slots.tolist() == [4, 2, 7] and ctx.want_rows.tolist() == [0, 2, 5]
    assert ctx.page_tables[0].tolist() == rows[0]
    assert (plan.max_new_tokens, plan.max_ctx_len, plan.is_decode) == (3, 132, False)
    for off in (plan.layout.positions, plan.layout.cu_seqlens, plan.layout.tables):
        assert off % 4 == 0
    with pytest.raises(ValueError, match="outside"):
        plan_step([SequenceStep(0, [1], want=[1])], [0], [[[0]]], 1)
    with pytest.raises(ValueError, match="at least one token"):
        plan_step([SequenceStep(0, [], want=[])], [0], [[[0]]], 1)


def test_window_groups_are_sized_by_their_window_when_steps_are_bounded():
    """With no step bringing a sequence more than 32 tokens, a group that keeps the last 40
    positions never holds more than 3 pages of a sequence, whatever its length, and its pool is
    that small; the group that keeps everything is sized by max_tokens.  Values may be narrower
    or wider than keys."""
    from wpc_engine_b200.cache.kv_cache import window_pages
    specs = [KVSpec(2, 16), KVSpec(2, 16, 40), KVSpec(1, 32, None, v_head_dim=8)]
    c = SequenceCache(specs, 64 * 50, torch.float32, "cpu", max_sequences=4, max_step_tokens=32)
    full, windowed, narrow = (c.groups[c.layer_group[i]] for i in range(3))
    assert window_pages(40, 32) == 3 and windowed.n_pages == 12 and full.n_pages == 50
    assert narrow.k.shape == (1, 50, 1, PAGE, 32) and narrow.v.shape == (1, 50, 1, PAGE, 8)
    slots = [c.open() for _ in range(4)]
    for step in range(40):                       # every sequence grows to 1,280 positions, 32 a step
        for s in slots[:1]:
            c.reserve(s, 32)
            assert sum(p >= 0 for p in windowed.tables[s]) <= 3
            c.commit(s, 32)
        c.check()
    assert windowed.pool.n_held <= 3 and full.pool.n_held == 20
    # what fits: the window group counts at most 3 pages a sequence, the full group all of them
    assert c.fits([1280, 640, 640, 640]) and not c.fits([1280, 1280, 640, 64])      # 51 pages in the full group
    assert not c.fits([1, 1, 1, 1, 1])                                               # five sequences, four slots
    unbounded = SequenceCache(specs, 64 * 50, torch.float32, "cpu", max_sequences=4)
    assert unbounded.groups[unbounded.layer_group[1]].n_pages == 50


def test_a_model_without_keys_and_values_has_no_page_budget():
    c = SequenceCache([StateSpec((4,)), None], 64, torch.float32, "cpu", max_sequences=3)
    assert c.kv_groups() == [] and c.fits([10 ** 6, 10 ** 6, 5]) and not c.fits([1] * 4)
    s = c.open()
    assert c.reserve(s, 10 ** 6) == 0
    c.commit(s, 10 ** 6)
    c.close(s)
    c.check()


def test_a_step_that_did_not_run_gives_its_pages_back():
    c = make_cache()
    a = c.open()
    c.reserve(a, 70)
    c.commit(a, 70)
    held = [g.pool.n_held for g in c.groups if isinstance(g, KVGroup)]
    c.reserve(a, 300)
    assert [g.pool.n_held for g in c.groups if isinstance(g, KVGroup)] != held
    c.release_unused(a)
    assert [g.pool.n_held for g in c.groups if isinstance(g, KVGroup)] == held and c.length(a) == 70
    c.check()
    c.close(a)
    assert all(g.pool.n_held == 0 for g in c.groups if isinstance(g, KVGroup))
