"""The engine: a model, its cache, and the one step function that everything above uses.

`step` takes a batch of sequences, each with the tokens it brings now (a whole prompt, a
chunk of one, or a single decoded token), runs exactly those tokens as one packed batch
against the cache, and returns the float32 logits at the wanted places.  The reference's
counterpart is `forward_token` (wpc-runtime/src/model.rs:419), one token of one sequence at a
time; batches, chunks and wanted places have no counterpart there.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from .. import ops
from ..cache import PAGE, CacheError, SequenceCache
from ..registry import config_from_folder, resolve
from ..weights import load_weights, random_weights_on_device
from .batch import SequenceStep, StepLayout, context_from, plan_step

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


def parse_dtype(dtype) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError(f"dtype must be bfloat16 or float32, got {dtype}")
        return dtype
    try:
        return _DTYPES[str(dtype)]
    except KeyError:
        raise ValueError(f"dtype must be bfloat16 or float32, got {dtype!r}") from None


def _bucket(n: int, floor: int = 4) -> int:
    b = floor
    while b < n:
        b *= 2
    return b


class _MetaRing:
    """Pinned host buffers for step metadata, reused in turn; a buffer is rewritten only after
    the copy that last read it has finished."""

    def __init__(self, device, depth: int = 4):
        self.device = torch.device(device)
        self.depth = depth
        self.bufs: List[Optional[torch.Tensor]] = [None] * depth
        self.events: List[Optional[object]] = [None] * depth
        self.i = 0
        self.pinned = self.device.type == "cuda"

    def next(self, n: int) -> torch.Tensor:
        self.i = (self.i + 1) % self.depth
        if self.events[self.i] is not None:
            self.events[self.i].synchronize()
        buf = self.bufs[self.i]
        if buf is None or buf.numel() < n:
            buf = torch.empty(max(n, 1024), dtype=torch.int32, pin_memory=self.pinned)
            self.bufs[self.i] = buf
        return buf

    def sent(self) -> None:
        if self.pinned:
            ev = torch.cuda.Event()
            ev.record()
            self.events[self.i] = ev


class Engine:
    """max_tokens: the most positions that live sequences hold at any time, each sequence
    rounded up to whole pages of 64; it sizes the cache.  use_graphs: replay single-token
    steps from CUDA graphs (one per batch size and page-table width).  max_step_tokens: the
    most tokens that one sequence may bring in one step (None: any number); with it, cache
    groups that keep a window are sized by the window.  check_status: `step` reads the device
    error word after it has run (which waits for the device) and raises `KernelError` if a
    kernel gave up; callers that keep the device busy pass `check=False` to `step` and read the
    word with their results (`generate` does).

    The limits of a step come from the model: `model.vocab_size` and `model.max_positions`."""

    def __init__(self, model, dtype, device="cuda", max_tokens: int = 4096,
                 max_sequences: Optional[int] = None, use_graphs: bool = True,
                 max_step_tokens: Optional[int] = None, check_status: bool = True):
        self.model = model
        self.config = model.config
        self.dtype = parse_dtype(dtype)
        self.device = torch.device(device)
        if max_step_tokens is not None and max_step_tokens < 1:
            raise ValueError(f"max_step_tokens must be at least 1, got {max_step_tokens}")
        self.max_step_tokens = max_step_tokens
        self.cache = SequenceCache(model.cache_specs(), max_tokens, self.dtype, self.device, max_sequences,
                                   max_step_tokens)
        self._ring = _MetaRing(self.device)
        self.use_graphs = bool(use_graphs) and self.device.type == "cuda" and model.graph_safe()
        self.check_status = bool(check_status) and self.device.type == "cuda"
        self._graphs: Dict[tuple, object] = {}
        self.vocab_size = model.vocab_size
        self.max_positions = model.max_positions
        if self.device.type == "cuda":
            # parameters are final from here on: kernels may fetch them ahead of their turn
            torch.cuda.synchronize(self.device)
        self._slot_tensors: Dict[tuple, torch.Tensor] = {}
        self._sampler_slots = set()     # slots whose sampler state was written since they were opened
        self.supports_device_tokens = self.device.type == "cuda"   # generation may queue a step ahead
        self.steps_run = 0
        self.graph_launches = 0      # kernels that graph replays have launched so far

    # -- construction ------------------------------------------------------------------------
    @classmethod
    def from_folder(cls, folder: str, dtype="bfloat16", device="cuda", **kw) -> "Engine":
        """A model folder: config.json names the architecture, model.safetensors holds the
        tensors."""
        ops.require_device(device)
        arch, config = config_from_folder(folder)
        model = arch.build(config)
        load_weights(model, folder, parse_dtype(dtype), torch.device(device))
        return cls(model, dtype, device, **kw)

    @classmethod
    def from_random(cls, config, seed: int = 0, dtype="bfloat16", device="cuda", **kw) -> "Engine":
        """Random weights drawn on the device (no folder); `config` is a configuration object
        of a registered architecture."""
        ops.require_device(device)
        model = resolve(config.to_dict()).build(config)
        random_weights_on_device(model, seed, parse_dtype(dtype), torch.device(device))
        return cls(model, dtype, device, **kw)

    # -- sequences ---------------------------------------------------------------------------
    def open_sequence(self) -> int:
        slot = self.cache.open()
        self._sampler_slots.discard(slot)      # the slot's last occupant left its seed and counter behind
        return slot

    def close_sequence(self, slot: int) -> None:
        self.cache.close(slot)
        self._sampler_slots.discard(slot)

    def sequence_length(self, slot: int) -> int:
        return self.cache.length(slot)

    # -- the step ----------------------------------------------------------------------------
    def _check(self, entries: Sequence[SequenceStep]) -> None:
        seen = set()
        for e in entries:
            if e.slot in seen:
                raise ValueError(f"slot {e.slot} appears twice in one step")
            seen.add(e.slot)
            if e.slot not in self.cache.lengths:
                raise CacheError(f"slot {e.slot} is not open")
            toks = np.asarray(e.tokens)
            if toks.size == 0:
                raise ValueError("every sequence of a step brings at least one token")
            if toks.min() < 0 or toks.max() >= self.vocab_size:
                raise ValueError(f"token id outside 0..{self.vocab_size - 1} in slot {e.slot}")
            if self.max_step_tokens is not None and toks.size > self.max_step_tokens:
                raise ValueError(f"slot {e.slot} brings {toks.size} tokens; this engine takes at most "
                                 f"{self.max_step_tokens} per sequence and step")
            end = self.cache.length(e.slot) + toks.size
            if self.max_positions is not None and end > self.max_positions:
                raise ValueError(f"slot {e.slot} would reach {end} positions; "
                                 f"the model's longest sequence is {self.max_positions}")

    def room(self, slot: int) -> Optional[int]:
        """How many more tokens the sequence in `slot` may bring (None: no limit)."""
        return None if self.max_positions is None else self.max_positions - self.cache.length(slot)

    def step(self, entries: Sequence[SequenceStep], device_tokens: Optional[torch.Tensor] = None,
             borrow: bool = False, check: Optional[bool] = None) -> Optional[torch.Tensor]:
        """Runs the tokens that each entry brings, from the cache that earlier steps left;
        returns float32 logits [wanted places, vocab] in the order of the entries and of their
        `want` lists, or None if nothing is wanted.  The tensor is the caller's own, unless
        `borrow` is set: then it may be a buffer that the next step of the same shape
        overwrites (for callers that use it at once, as sampling does).

        `device_tokens` (int32 on the device, one per entry, for single-token steps): the
        token ids are taken from there instead of the entries', so that a step can be queued
        behind the sampling of its tokens without the host having seen them.

        `check` (default: the engine's `check_status`): read the device error word after the
        step, which waits for the device, and raise `KernelError` if a kernel of the step gave
        up.  A step that raises, for whatever reason, leaves the sequences as they were: the
        pages that it had taken go back."""
        self._check(entries)
        reserved = []
        try:
            starts = []
            for e in entries:
                reserved.append(e.slot)        # first: a sequence may have got pages in one group and none in the next
                starts.append(self.cache.reserve(e.slot, len(e.tokens)))
            logits = self._run(entries, starts, device_tokens, borrow)
            if self.check_status if check is None else check:
                ops.check_device_status(self.device, "a kernel of the step")
        except BaseException:
            for slot in reserved:
                self.cache.release_unused(slot)
            raise
        for e in entries:
            self.cache.commit(e.slot, len(e.tokens))
        self.steps_run += 1
        return logits

    def _run(self, entries, starts, device_tokens, borrow) -> Optional[torch.Tensor]:
        slots = [e.slot for e in entries]
        width = _bucket(self.cache.table_width(slots))
        kv_groups = self.cache.kv_groups()
        rows = [self.cache.page_table_rows(g, slots, width) for g in kv_groups]
        n_tokens = sum(len(e.tokens) for e in entries)
        n_want = sum(len(e.want) for e in entries)
        lay = StepLayout(n_tokens, len(entries), n_want, width, len(kv_groups))
        host = self._ring.next(lay.total)
        plan = plan_step(entries, starts, rows, width, out=host.numpy())
        logits = None
        ran = False
        if device_tokens is not None and not (plan.is_decode and device_tokens.numel() == len(entries)
                                              and device_tokens.dtype == torch.int32):
            raise ValueError("device_tokens needs a single-token step and one int32 id per entry")
        if plan.is_decode and self.use_graphs:
            ran, logits = self._graph_step(plan, host, device_tokens)
            if ran and logits is not None and not borrow:
                logits = logits.clone()        # the graph's own output buffer: the next replay overwrites it
        if not ran:
            meta = host[: lay.total].to(self.device, non_blocking=True)
            self._ring.sent()
            if device_tokens is not None:
                meta[lay.tokens: lay.tokens + lay.n_tokens].copy_(device_tokens)
            ctx = context_from(meta, lay, self.dtype, plan.max_new_tokens, plan.max_ctx_len, plan.is_decode,
                               [len(e.tokens) for e in entries])
            logits = self.model.forward(ctx, self.cache)
        return logits

    def _graph_step(self, plan, host: torch.Tensor, device_tokens: Optional[torch.Tensor] = None):
        """Single-token steps of a shape seen before are replayed from a CUDA graph.  The first
        step of a shape runs directly (returns ran=False); the second is captured, which runs
        nothing, and then replayed, so that no step ever runs twice."""
        lay = plan.layout
        key = (lay.n_seqs, lay.table_width, lay.n_want)
        entry = self._graphs.get(key)
        if entry is None:
            self._graphs[key] = "seen"
            return False, None
        if entry == "seen":
            meta = torch.zeros(lay.total, dtype=torch.int32, device=self.device)
            ctx = context_from(meta, lay, self.dtype, 1, lay.table_width * PAGE, True)
            graph = torch.cuda.CUDAGraph()
            before = ops.launch_count
            with torch.cuda.graph(graph):
                logits = self.model.forward(ctx, self.cache)
            entry = (graph, meta, logits, ops.launch_count - before)
            self._graphs[key] = entry
        graph, meta, logits, n_kernels = entry
        meta.copy_(host[: lay.total], non_blocking=True)
        self._ring.sent()
        if device_tokens is not None:
            meta[lay.tokens: lay.tokens + lay.n_tokens].copy_(device_tokens)
        graph.replay()
        self.graph_launches += n_kernels
        return True, logits

    # -- the device error word ------------------------------------------------------------------
    def status_word(self) -> Optional[torch.Tensor]:
        """int32 [1] on the device, non-zero once a kernel gave up (None without a device); for
        callers that copy it to the host beside their results instead of letting `step` wait."""
        return ops.status_word(self.device) if self.device.type == "cuda" else None

    def raise_status(self, code: int) -> None:
        """Raises `KernelError` for a non-zero status word that the caller has read, and clears it."""
        ops.raise_device_status(int(code), self.device, "a kernel of an earlier step")

    # -- sampling ----------------------------------------------------------------------------
    def set_sampler_state(self, slots: Sequence[int], seed: int, request_ids: Sequence[int]) -> None:
        """Writes (seed, request number, 0 tokens drawn) into the slots' state rows."""
        rows = torch.tensor([[0, seed, r, 0] for r in request_ids], dtype=torch.int64)
        idx = torch.tensor(list(slots), dtype=torch.int64)
        self.cache.seq_state[idx.to(self.device)] = rows.to(self.device)
        self._sampler_slots.update(int(s) for s in slots)

    def sample(self, logits: torch.Tensor, slots: Sequence[int], temperature: float,
               banned: Sequence[int] = ()) -> torch.Tensor:
        """One token per row of `logits`, int32 on the device; row i belongs to slots[i].  A draw
        with a temperature needs the slots' sampler state (`set_sampler_state`) written since
        they were opened: a slot keeps its last occupant's seed and counter otherwise."""
        if temperature > 0:
            unset = [s for s in slots if s not in self._sampler_slots]
            if unset:
                raise ValueError(f"slots {unset} have no sampler state: call set_sampler_state after open_sequence")
        key = tuple(slots)
        slot_t = self._slot_tensors.get(key)
        if slot_t is None:
            if len(self._slot_tensors) > 256:
                self._slot_tensors.clear()
            slot_t = torch.tensor(list(slots), dtype=torch.int32).to(self.device)
            self._slot_tensors[key] = slot_t
        banned_t = None
        if len(banned):
            banned_t = torch.tensor(sorted(set(int(b) for b in banned)), dtype=torch.int32).to(self.device)
        return ops.sample(logits, slot_t, self.cache.seq_state, float(temperature), banned_t)
