"""Helpers shared by the tests: running requests through an engine in the three ways that the
comparisons need, and reading the plain implementation's answers."""
import numpy as np
import torch

from plain import qwen2_plain as P
from wpc_engine_b200 import SequenceStep


def plain_logits(folder, tokens, dtype=np.float64):
    cfg, tensors = P.read_model_folder(folder)
    return P.forward(cfg, tensors, tokens, dtype)


def random_tokens(vocab, n, seed):
    rng = np.random.default_rng(seed)
    return rng.integers(0, vocab, size=n).tolist()


def run_whole(engine, tokens):
    """One request alone, all tokens in one step, logits at every place: [T, V]."""
    slot = engine.open_sequence()
    try:
        out = engine.step([SequenceStep(slot, tokens, want=list(range(len(tokens))))])
        return out.float().cpu().numpy()
    finally:
        engine.close_sequence(slot)


def run_tail_one_by_one(engine, tokens, tail=32):
    """The first T - tail tokens in one step, the last `tail` one token a step: [T, V]."""
    slot = engine.open_sequence()
    try:
        head = max(len(tokens) - tail, 0)
        rows = []
        if head:
            rows.append(engine.step([SequenceStep(slot, tokens[:head], want=list(range(head)))]).float().cpu().numpy())
        for t in tokens[head:]:
            rows.append(engine.step([SequenceStep(slot, [t], want=[0])]).float().cpu().numpy())
        return np.concatenate(rows, axis=0)
    finally:
        engine.close_sequence(slot)


def run_batch(engine, requests, prompt_lens):
    """Requests that start together: request i brings prompt_lens[i] tokens in the first step
    and then one token a step until its own end, leaving the batch when it has none left.
    Returns the logits of every place of every request: list of [T_i, V]."""
    slots = [engine.open_sequence() for _ in requests]
    rows = [[] for _ in requests]
    try:
        entries = [SequenceStep(s, r[:n], want=list(range(n))) for s, r, n in zip(slots, requests, prompt_lens)]
        fed = list(prompt_lens)
        live = list(range(len(requests)))
        while live:
            out = engine.step(entries).float().cpu().numpy()
            at = 0
            for i, e in zip(live, entries):
                rows[i].append(out[at: at + len(e.want)])
                at += len(e.want)
            still = []
            for i in live:
                if fed[i] < len(requests[i]):
                    still.append(i)
                else:
                    engine.close_sequence(slots[i])
                    slots[i] = None
            live = still
            entries = [SequenceStep(slots[i], [requests[i][fed[i]]], want=[0]) for i in live]
            for i in live:
                fed[i] += 1
        return [np.concatenate(r, axis=0) for r in rows]
    finally:
        for s in slots:
            if s is not None:
                engine.close_sequence(s)


def bfloat16_bound(want64):
    """The largest error allowed to bfloat16 logits against the plain implementation in
    float64, fixed here once for all tests: three times the largest error that the engine showed
    on the tiny configurations (whole, tail one by one, batches, mixed steps: 0.21 of
    0.03 std + 0.02 max when this was set), in units of the logits' spread and size."""
    return 0.02 * want64.std() + 0.012 * np.abs(want64).max()


def assert_close_to_plain(got, folder, tokens, dtype_name, what=""):
    """Compares engine logits [T, V] with the plain implementation in float64.

    float32: the error may be a few times the plain implementation's own float32 rounding
    noise against float64.  bfloat16: `bfloat16_bound`."""
    want64 = plain_logits(folder, tokens, np.float64)
    err = np.abs(got.astype(np.float64) - want64).max()
    if dtype_name == "float32":
        want32 = plain_logits(folder, tokens, np.float32)
        noise = np.abs(want32.astype(np.float64) - want64).max()
        bound = 4 * noise + 1e-6
    else:
        bound = bfloat16_bound(want64)
    assert err <= bound, f"{what}: max error {err:.3e} exceeds {bound:.3e}"
    return err
