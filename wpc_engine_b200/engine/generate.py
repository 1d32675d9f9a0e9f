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
from typing import Callable, List, Optional, Sequence, Union

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


def plan_batches(prompt_lens: Sequence[int], max_tokens: int, room: Union[int, None, Callable[[List[int]], bool]],
                 n_slots: int, max_batch: Optional[int] = None) -> List[List[int]]:
    """Request numbers grouped into batches, in order.  A batch takes requests while every one
    of them can reach prompt + max_tokens positions within the cache and its slots.

    `room` says what fits: a number of pages of 64 positions that all sequences of a batch
    share; None for a model that keeps no keys and values (only slots limit a batch); or a
    function that takes the final lengths of a batch's sequences and answers whether the cache
    holds them all at once (`SequenceCache.fits`, which knows every group's own pool)."""
    if room is None:
        def fits(lens):
            return True
    elif callable(room):
        fits = room
    else:
        def fits(lens):
            return sum(pages_for(n) for n in lens) <= room
    batches: List[List[int]] = []
    cur: List[int] = []
    cur_lens: List[int] = []
    limit = min(n_slots, max_batch) if max_batch else n_slots
    for r, n in enumerate(prompt_lens):
        if n < 1:
            raise ValueError(f"request {r} has an empty prompt")
        total = n + max_tokens
        if not fits([total]):
            raise ValueError(f"request {r} needs {pages_for(total)} pages of 64 positions ({n} prompt + "
                             f"{max_tokens} new); the cache does not hold that many")
        if cur and (len(cur) >= limit or not fits(cur_lens + [total])):
            batches.append(cur)
            cur, cur_lens = [], []
        cur.append(r)
        cur_lens.append(total)
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


def prompt_steps(slots: Sequence[int], prompts: Sequence[Sequence[int]],
                 chunk: Optional[int]) -> List[List[SequenceStep]]:
    """The steps that feed the prompts of a batch.  Without `chunk`: one step with every whole
    prompt, the last place of each wanted.  With it, no sequence brings more than `chunk`
    tokens a step: step i carries tokens i*chunk .. of every prompt that has any left, and a
    prompt's last place is wanted in the step that carries it (sequences with short prompts
    then wait for the long ones before they are fed their first drawn token)."""
    if not chunk:
        return [[SequenceStep(s, list(p), want=[len(p) - 1]) for s, p in zip(slots, prompts)]]
    steps = []
    at = 0
    while any(at < len(p) for p in prompts):
        entries = []
        for s, p in zip(slots, prompts):
            part = list(p[at: at + chunk])
            if part:
                entries.append(SequenceStep(s, part, want=[len(part) - 1] if at + chunk >= len(p) else []))
        steps.append(entries)
        at += chunk
    return steps


def _first_logits(engine, live, steps, stats, **step_args):
    """Feeds the prompt steps; returns the logits of every sequence's last prompt place in the
    order of `live`, the entries of the last step, and when that step began (the caller notes
    it once its tokens are drawn; the earlier ones are noted here)."""
    t0 = time.perf_counter()
    if len(steps) == 1:
        return engine.step(steps[0], **step_args), steps[0], t0
    import torch
    rows = {}
    for entries in steps:
        t0 = time.perf_counter()
        logits = engine.step(entries, **step_args)
        at = 0
        for e in entries:
            if len(e.want):
                rows[e.slot] = logits[at: at + 1].clone()
                at += 1
        if entries is not steps[-1]:
            _note(stats, True, time.perf_counter() - t0, entries)
    return torch.cat([rows[s.slot] for s in live], dim=0), steps[-1], t0


def _run_batch(engine, live, steps, opts, stop, outputs, stats) -> None:
    """One batch, step by step: every step waits for its tokens on the host."""
    first = True
    logits, entries, t0 = _first_logits(engine, live, steps, stats)
    while live:
        if logits is None:
            t0 = time.perf_counter()
            logits = engine.step(entries)
        picked = engine.sample(logits, [s.slot for s in live], opts.temperature,
                               opts.banned_token_ids).tolist()      # the step's one device-to-host read
        logits = None
        _note(stats, first, time.perf_counter() - t0, entries)
        first = False
        live[:], done = advance(live, picked, opts, stop)
        for seq in done:
            outputs[seq.request] = seq.output
            engine.close_sequence(seq.slot)
        entries = [SequenceStep(s.slot, [s.output[-1]], want=[0]) for s in live]


class _HostRead:
    """The step's one device-to-host read: the sampled ids and, behind them, the device error
    word, copied into one pinned buffer; `wait` returns once both have arrived."""

    def __init__(self, engine, n: int):
        import torch
        self.torch = torch
        self.cuda = engine.device.type == "cuda"
        self.status = engine.status_word() if hasattr(engine, "status_word") else None
        self.buf = torch.empty(n + 1, dtype=torch.int32, pin_memory=self.cuda)   # pageable memory would make the copy block
        self.index_cache = {}
        self.event = None

    def start(self, ids) -> None:
        n = ids.numel()
        self.n = n
        self.buf[:n].copy_(ids, non_blocking=True)
        if self.status is not None:
            self.buf[n: n + 1].copy_(self.status, non_blocking=True)
        else:
            self.buf[n] = 0
        if self.cuda:
            self.event = self.torch.cuda.Event()
            self.event.record()

    def wait(self):
        """(ids as a list, status word)"""
        if self.event is not None:
            self.event.synchronize()
        return self.buf[: self.n].tolist(), int(self.buf[self.n])

    def index(self, places: Sequence[int], device):
        """`places` as an index tensor on the device, copied from pinned memory (the copy of a
        pageable tensor would stall the host until the stream has drained); kept per set."""
        key = tuple(places)
        got = self.index_cache.get(key)
        if got is None:
            host = self.torch.tensor(list(places), dtype=self.torch.int64)
            if self.cuda:
                host = host.pin_memory()
            got = (host.to(device, non_blocking=True), host)   # the pinned source lives as long as the copy may run
            self.index_cache[key] = got
        return got[0]


def _run_batch_pipelined(engine, live, steps, opts, stop, outputs, stats) -> None:
    """One batch with the next step queued before the host has read the current tokens: the
    sampled ids stay on the device and feed the next step from there, so the device never
    waits for the host.  Who ends by reaching max_tokens is known in advance and gets no
    further step, and neither does a sequence that has no room for another token: whether
    that is an error is decided when the host has seen that its token was no stop token.  A
    stop token is only seen one step late: that sequence has then run one step too many, whose
    result is dropped (its slot is closed behind that step in stream order).  The tokens that
    come out are the same as step by step.  The device error word travels with the ids; a
    kernel that gave up ends the batch with `KernelError`."""
    first = True
    logits, entries, t0 = _first_logits(engine, live, steps, stats, borrow=True, check=False)
    read = _HostRead(engine, len(live))
    room_of = getattr(engine, "room", None)
    while live:
        ids = engine.sample(logits, [s.slot for s in live], opts.temperature, opts.banned_token_ids)
        read.start(ids)
        # who would go on if the token just drawn is no stop token
        wants = [i for i, s in enumerate(live) if len(s.output) + 1 < opts.max_tokens]
        full = [i for i in wants if room_of is not None and room_of(live[i].slot) is not None
                and room_of(live[i].slot) < 1]
        ahead = [i for i in wants if i not in full]
        next_logits = None
        next_entries = []
        if ahead:
            next_entries = [SequenceStep(live[i].slot, [0], want=[0]) for i in ahead]
            feed = ids if len(ahead) == len(live) else ids[read.index(ahead, ids.device)]
            next_logits = engine.step(next_entries, device_tokens=feed, borrow=True, check=False)
        picked, status = read.wait()                  # the step's one device-to-host read
        if status:
            engine.raise_status(status)
        now = time.perf_counter()
        _note(stats, first, now - t0, entries)
        t0, first, entries = now, False, next_entries
        ahead_seqs = [live[i] for i in ahead]
        full_seqs = [live[i] for i in full]
        go_on, done = advance(live, picked, opts, stop)
        for seq in full_seqs:
            if any(seq is g for g in go_on):
                raise ValueError(f"request {seq.request} has reached the model's longest sequence "
                                 f"({engine.max_positions} positions) and its last token is no stop token")
        for seq in done:
            outputs[seq.request] = seq.output
            engine.close_sequence(seq.slot)
        if len(go_on) != len(ahead_seqs):
            # some of those that ran ahead met a stop token: drop their rows
            keep = [i for i, s in enumerate(ahead_seqs) if any(s is g for g in go_on)]
            next_logits = next_logits[read.index(keep, next_logits.device)] if keep else None
        live[:] = go_on
        logits = next_logits


def generate(engine, prompts: Sequence[Sequence[int]], opts: GenerationOptions,
             stats: Optional[dict] = None) -> List[List[int]]:
    """Generated token ids for each prompt.  `engine` offers open_sequence, close_sequence,
    step, sample, set_sampler_state and a `cache` with n_slots and either `fits` (see
    plan_batches) or n_pages.  An engine with `max_step_tokens` gets its prompts in chunks of
    that many tokens.

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
    room = getattr(engine.cache, "fits", None) or engine.cache.n_pages
    batches = plan_batches([len(p) for p in prompts], opts.max_tokens, room, engine.cache.n_slots, opts.max_batch)
    chunk = getattr(engine, "max_step_tokens", None)
    for batch in batches:
        live = [_Live(r, engine.open_sequence()) for r in batch]
        try:
            engine.set_sampler_state([s.slot for s in live], opts.seed, [s.request for s in live])
            steps = prompt_steps([s.slot for s in live], [prompts[s.request] for s in live], chunk)
            if getattr(engine, "supports_device_tokens", False):
                _run_batch_pipelined(engine, live, steps, opts, stop, outputs, stats)
            else:
                _run_batch(engine, live, steps, opts, stop, outputs, stats)
            live = []
        except BaseException:
            for seq in live:
                try:
                    engine.close_sequence(seq.slot)
                except Exception:
                    pass
            raise
    return [o if o is not None else [] for o in outputs]
