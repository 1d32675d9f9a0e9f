"""The generation loop above the step function: batches of unequal prompts, stop tokens,
sequences that end earlier, and as many batches one after another as there are requests.

The order within a sequence is the reference's (wpc-runtime/src/main.rs:284-312): pick a
token from the last logits, append it, stop if it is a stop token (it stays in the output and
is never fed), else feed it.  The forward pass that the reference spends after the last
token (main.rs:307) is not run.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

from ..cache import pages_for
from .batch import SequenceStep


@dataclass
class GenerationOptions:
    max_tokens: int = 40                    # main.rs:61-62
    temperature: float = 0.0                # 0: greedy (sampling.rs:3-13)
    seed: int = 0
    stop_token_ids: Sequence[int] = ()
    banned_token_ids: Sequence[int] = ()    # sampling.rs:23-51 (WPC_BAN_TOKENS)
    max_batch: Optional[int] = None         # most sequences in one batch


def plan_batches(prompt_lens: Sequence[int], max_tokens: int, n_pages: int, n_slots: int,
                 max_batch: Optional[int] = None) -> List[List[int]]:
    """Request numbers grouped into batches, in order.  A batch takes requests while every one
    of them can reach prompt + max_tokens positions within the cache's pages and slots."""
    batches: List[List[int]] = []
    cur: List[int] = []
    cur_pages = 0
    limit = min(n_slots, max_batch) if max_batch else n_slots
    for r, n in enumerate(prompt_lens):
        if n < 1:
            raise ValueError(f"request {r} has an empty prompt")
        need = pages_for(n + max_tokens)
        if need > n_pages:
            raise ValueError(f"request {r} needs {need} pages of 64 positions ({n} prompt + {max_tokens} new); "
                             f"the cache has {n_pages}")
        if cur and (cur_pages + need > n_pages or len(cur) >= limit):
            batches.append(cur)
            cur, cur_pages = [], 0
        cur.append(r)
        cur_pages += need
    if cur:
        batches.append(cur)
    return batches


@dataclass
class _Live:
    request: int
    slot: int
    output: List[int] = field(default_factory=list)


def advance(live: List[_Live], picked: Sequence[int], opts: GenerationOptions, stop: frozenset):
    """Appends each picked token to its sequence and decides who goes on: returns (still
    live, finished).  A sequence ends on a stop token or when it has max_tokens tokens."""
    go_on, done = [], []
    for seq, tok in zip(live, picked):
        tok = int(tok)
        seq.output.append(tok)
        if tok in stop or len(seq.output) >= opts.max_tokens:
            done.append(seq)
        else:
            go_on.append(seq)
    return go_on, done


def _note(stats, first: bool, dt: float, entries) -> None:
    if stats is None:
        return
    if first:
        stats["prefill_s"] += dt
        stats["prefill_tokens"] += sum(len(e.tokens) for e in entries)
    else:
        stats["decode_s"] += dt
        stats["decode_tokens"] += len(entries)
        stats["decode_steps"] += 1
        stats["decode_step_s"].append(dt)
        stats["decode_step_tokens"].append(len(entries))


def _run_batch(engine, live, entries, opts, stop, outputs, stats) -> None:
    """One batch, step by step: every step waits for its tokens on the host."""
    first = True
    while live:
        t0 = time.perf_counter()
        logits = engine.step(entries)
        picked = engine.sample(logits, [s.slot for s in live], opts.temperature,
                               opts.banned_token_ids).tolist()      # the step's one device-to-host read
        _note(stats, first, time.perf_counter() - t0, entries)
        first = False
        live[:], done = advance(live, picked, opts, stop)
        for seq in done:
            outputs[seq.request] = seq.output
            engine.close_sequence(seq.slot)
        entries = [SequenceStep(s.slot, [s.output[-1]], want=[0]) for s in live]


def _run_batch_pipelined(engine, live, entries, opts, stop, outputs, stats) -> None:
    """One batch with the next step queued before the host has read the current tokens: the
    sampled ids stay on the device and feed the next step from there, so the device never
    waits for the host.  Who ends by reaching max_tokens is known in advance and gets no
    further step.  A stop token is only seen one step late: that sequence has then run one
    step too many, whose result is dropped (its slot is closed behind that step in stream
    order).  The tokens that come out are the same as step by step."""
    import torch
    first = True
    t0 = time.perf_counter()
    logits = engine.step(entries)
    pinned = torch.empty(len(live), dtype=torch.int32, pin_memory=True)   # pageable memory would make the copy block
    while live:
        ids = engine.sample(logits, [s.slot for s in live], opts.temperature, opts.banned_token_ids)
        host_ids = pinned[: len(live)]
        host_ids.copy_(ids, non_blocking=True)
        done_event = torch.cuda.Event()
        done_event.record()
        # who would go on if the token just drawn is no stop token
        ahead = [i for i, s in enumerate(live) if len(s.output) + 1 < opts.max_tokens]
        next_logits = None
        next_entries = []
        if ahead:
            next_entries = [SequenceStep(live[i].slot, [0], want=[0]) for i in ahead]
            feed = ids if len(ahead) == len(live) else ids[torch.tensor(ahead, device=ids.device)]
            next_logits = engine.step(next_entries, device_tokens=feed)
        done_event.synchronize()                      # the step's one device-to-host read
        picked = host_ids.tolist()
        now = time.perf_counter()
        _note(stats, first, now - t0, entries)
        t0, first, entries = now, False, next_entries
        ahead_seqs = [live[i] for i in ahead]
        go_on, done = advance(live, picked, opts, stop)
        for seq in done:
            outputs[seq.request] = seq.output
            engine.close_sequence(seq.slot)
        if len(go_on) != len(ahead_seqs):
            # some of those that ran ahead met a stop token: drop their rows
            keep = [i for i, s in enumerate(ahead_seqs) if any(s is g for g in go_on)]
            next_logits = next_logits[torch.tensor(keep, device=next_logits.device)] if keep else None
        live[:] = go_on
        logits = next_logits


def generate(engine, prompts: Sequence[Sequence[int]], opts: GenerationOptions,
             stats: Optional[dict] = None) -> List[List[int]]:
    """Generated token ids for each prompt.  `engine` offers open_sequence, close_sequence,
    step, sample, set_sampler_state and a `cache` with n_pages and n_slots.

    With `stats` (a dict) the loop records what the reference prints to standard error
    (wpc-runtime/src/main.rs:294, 309): seconds and tokens of the prompt steps and of the
    single-token steps, summed over the batches; `decode_step_s` and `decode_step_tokens` list
    the seconds and tokens of every single-token step in order."""
    if opts.max_tokens < 1:
        return [[] for _ in prompts]
    if stats is not None:
        stats.update(prefill_s=0.0, prefill_tokens=0, decode_s=0.0, decode_tokens=0, decode_steps=0,
                     decode_step_s=[], decode_step_tokens=[])
    stop = frozenset(int(s) for s in opts.stop_token_ids)
    outputs: List[Optional[List[int]]] = [None] * len(prompts)
    batches = plan_batches([len(p) for p in prompts], opts.max_tokens, engine.cache.n_pages,
                           engine.cache.n_slots, opts.max_batch)
    for batch in batches:
        live = [_Live(r, engine.open_sequence()) for r in batch]
        try:
            engine.set_sampler_state([s.slot for s in live], opts.seed, [s.request for s in live])
            entries = [SequenceStep(s.slot, list(prompts[s.request]), want=[len(prompts[s.request]) - 1])
                       for s in live]
            if getattr(engine, "supports_device_tokens", False):
                _run_batch_pipelined(engine, live, entries, opts, stop, outputs, stats)
            else:
                _run_batch(engine, live, entries, opts, stop, outputs, stats)
            live = []
        except BaseException:
            for seq in live:
                try:
                    engine.close_sequence(seq.slot)
                except Exception:
                    pass
            raise
    return [o if o is not None else [] for o in outputs]
