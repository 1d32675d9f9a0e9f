"""Each part of a layer alone on the GPU against the plain implementation's function for it,
at sizes of its own, and two toy architectures: one with a mixer that keeps a state of fixed
size per sequence (and a layer scheduled twice), one with a feed-forward that routes each token
to one of several experts in some of its layers and with a position encoding of its own.  Both
are registered, built, written, loaded and stepped from the tests, without a change to the
library's files."""
import dataclasses
import json
import math
import os

import numpy as np
import pytest
import torch

from plain import qwen2_plain as P
import wpc_engine_b200 as wpc
from wpc_engine_b200.cache import SequenceCache
from wpc_engine_b200.engine.batch import SequenceStep, context_from, plan_step
from wpc_engine_b200.models.decoder import DecoderModel, Run
from wpc_engine_b200.parts import (Embedding, GQAAttention, Linear, Mixer, OutputHead, ParamSpec, PreNormBlock,
                                   RMSNorm, RotaryEncoding, StateSpec, SwiGLU)
from wpc_engine_b200.weights.loader import bind_model, finalize_parts

pytestmark = pytest.mark.gpu
DEV = "cuda"


def rnd(shape, seed, scale=1.0):
    return (torch.randn(shape, generator=torch.Generator().manual_seed(seed)) * scale)


def make_ctx(dtype, lens_new, starts, cache=None, slots=None):
    """A step context for sequences that bring lens_new[b] tokens after starts[b] cached ones."""
    entries = [SequenceStep(slots[b] if slots else b, [1] * n, want=[n - 1]) for b, n in enumerate(lens_new)]
    rows, width = [], 1
    if cache is not None:
        width = cache.table_width([e.slot for e in entries])
        rows = [cache.page_table_rows(g, [e.slot for e in entries], width) for g in cache.kv_groups()]
    plan = plan_step(entries, starts, rows, width)
    meta = torch.from_numpy(plan.host).to(DEV)
    return context_from(meta, plan.layout, dtype, plan.max_new_tokens, plan.max_ctx_len, plan.is_decode, list(lens_new))


def bind(part, tensors, dtype):
    from wpc_engine_b200.parts.base import collect_params
    from wpc_engine_b200.weights.loader import device_dtype
    wanted = collect_params(part)
    per = {}
    for name, (owner, local, spec) in wanted.items():
        t = tensors[name]
        per.setdefault(id(owner), (owner, {}))[1][local] = t.to(DEV, device_dtype(t.dtype, spec.kind, dtype)).contiguous()
    for owner, d in per.values():
        owner.bind(d)
    finalize_parts(part)


def tol(dtype):
    return 3e-5 if dtype == torch.float32 else 2e-2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_part(dtype):
    part = RMSNorm(88, 3e-5)
    g = 1 + rnd((88,), 1, 0.1)
    bind(part, {"weight": g}, dtype)
    x = rnd((7, 88), 2, 2.0)
    got = part.forward(make_ctx(dtype, [7], [0]), x.to(DEV))
    want = P.rms_norm(x.numpy().astype(np.float64), g.numpy().astype(np.float64), 3e-5)
    assert np.abs(got.float().cpu().numpy() - want).max() <= tol(dtype) * np.abs(want).max()


def test_rotary_part_shares_tables_and_handles_partial_rotation():
    rot = RotaryEncoding(32, 1e4, rotary_pairs=10)
    ctx = make_ctx(torch.float32, [3, 2], [5, 0])
    cos, sin = rot.tables(ctx)
    assert rot.tables(ctx)[0] is cos and cos.shape == (5, 10)          # computed once per step
    x = rnd((5, 2 * 32), 3).to(DEV)
    y = wpc.ops.rope_inplace(x.clone(), 2, 32, cos, sin)
    pos = [5, 6, 7, 0, 1]
    xv = x.cpu().numpy().astype(np.float64).reshape(5, 2, 32)
    i = np.arange(10)
    ang = np.asarray(pos)[:, None] * np.power(1e4, -2.0 * i / 32)[None, :]
    want = xv.copy()
    want[..., :10] = xv[..., :10] * np.cos(ang)[:, None] - xv[..., 16:26] * np.sin(ang)[:, None]
    want[..., 16:26] = xv[..., 16:26] * np.cos(ang)[:, None] + xv[..., :10] * np.sin(ang)[:, None]
    assert np.abs(y.cpu().numpy().reshape(5, 2, 32) - want).max() < 1e-5
    assert torch.equal(y[3], x[3])                                      # position 0 is the identity


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_feed_forward_part(dtype):
    part = SwiGLU(72, 200)
    ts = {"gate_proj.weight": rnd((200, 72), 4, 0.1), "up_proj.weight": rnd((200, 72), 5, 0.1),
          "down_proj.weight": rnd((72, 200), 6, 0.1)}
    ts = {k: v.to(dtype) for k, v in ts.items()}
    bind(part, ts, dtype)
    h = rnd((9, 72), 7).to(dtype)
    residual = rnd((9, 72), 8).to(DEV)
    r0 = residual.clone()
    assert part.forward(make_ctx(dtype, [9], [0]), h.to(DEV), residual) is None
    f = lambda t: t.float().numpy().astype(np.float64)
    want = f(r0.cpu()) + P.swiglu(f(h), f(ts["gate_proj.weight"]), f(ts["up_proj.weight"]), f(ts["down_proj.weight"]))
    assert np.abs(residual.cpu().numpy() - want).max() <= tol(dtype) * np.abs(want).max()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [None, 20])
def test_attention_part_over_two_steps(dtype, window):
    """The mixer alone with a cache of its own: a prompt step, then a second step that brings
    more tokens; both against the plain attention over the whole sequence."""
    W, nh, nkv, hd = 56, 6, 2, 16
    rot = RotaryEncoding(hd, 1e4)
    part = GQAAttention(W, nh, nkv, hd, position=rot, qkv_bias=True, window=window)
    ts = {f"{n}_proj.weight": rnd((o, W), 10 + i, 0.2) for i, (n, o) in enumerate([("q", nh * hd), ("k", nkv * hd), ("v", nkv * hd)])}
    ts.update({f"{n}_proj.bias": rnd((o,), 20 + i, 0.2) for i, (n, o) in enumerate([("q", nh * hd), ("k", nkv * hd), ("v", nkv * hd)])})
    ts["o_proj.weight"] = rnd((W, nh * hd), 30, 0.2)
    ts = {k: v.to(dtype) for k, v in ts.items()}
    bind(part, ts, dtype)
    cache = SequenceCache([part.cache_spec()], 512, dtype, DEV)
    slot = cache.open()
    T1, T2 = 70, 9
    h = rnd((T1 + T2, W), 40).to(dtype)
    outs = []
    for lo, n in ((0, T1), (T1, T2)):
        cache.reserve(slot, n)
        ctx = make_ctx(dtype, [n], [lo], cache, [slot])
        model_stub = DecoderModel(None, Embedding(2, W), [PreNormBlock(RMSNorm(W, 1e-6), part, RMSNorm(W, 1e-6), SwiGLU(W, 8))],
                                  RMSNorm(W, 1e-6), OutputHead(2, W))
        view = model_stub.cache_views(cache, ctx)[0]
        residual = torch.zeros((n, W), dtype=torch.float32, device=DEV)
        part.forward(ctx, h[lo:lo + n].to(DEV), view, residual)
        outs.append(residual.cpu().numpy())
        cache.commit(slot, n)
    f = lambda t: t.float().numpy().astype(np.float64)
    hh = f(h)
    q = P.rope(P.linear(hh, f(ts["q_proj.weight"]), f(ts["q_proj.bias"])).reshape(-1, nh, hd), np.arange(T1 + T2), 1e4)
    k = P.rope(P.linear(hh, f(ts["k_proj.weight"]), f(ts["k_proj.bias"])).reshape(-1, nkv, hd), np.arange(T1 + T2), 1e4)
    v = P.linear(hh, f(ts["v_proj.weight"]), f(ts["v_proj.bias"])).reshape(-1, nkv, hd)
    want = P.linear(P.attention(q, k, v, window).reshape(-1, nh * hd), f(ts["o_proj.weight"]))
    got = np.concatenate(outs)
    assert np.abs(got - want).max() <= tol(dtype) * np.abs(want).max()


def test_embedding_and_heads():
    emb = Embedding(50, 24)
    table = rnd((50, 24), 50)
    bind(emb, {"weight": table}, torch.float32)
    ctx = make_ctx(torch.float32, [3], [0])
    ctx.tokens.copy_(torch.tensor([4, 49, 0], dtype=torch.int32))
    assert torch.equal(emb.forward(ctx).cpu(), table[[4, 49, 0]])
    tied = OutputHead(50, 24, tied_to=emb)
    assert tied.param_specs() == {}
    h = rnd((3, 24), 51).to(DEV)
    assert torch.allclose(tied.forward(ctx, h).cpu(), h.cpu() @ table.t(), atol=1e-5)
    own = OutputHead(50, 24)
    w = rnd((50, 24), 52)
    bind(own, {"weight": w}, torch.float32)
    assert torch.allclose(own.forward(ctx, h).cpu(), h.cpu() @ w.t(), atol=1e-5)


# ---- a toy architecture defined here: a mixer with a running state per sequence --------------------
class RunningMeanMixer(Mixer):
    """state <- decay * state + (1 - decay) * h_t for each token in order; out_t = W state.
    Keeps one [width] record per sequence; written with torch calls, since it is only a toy,
    and not capturable into a graph because it reads the slots on the host."""
    graph_safe = False

    def __init__(self, width, decay):
        self.width, self.decay = width, decay
        self.proj = Linear(width, width)

    def subparts(self):
        return {"proj": self.proj}

    def cache_spec(self):
        return StateSpec((self.width,), "float32")

    def forward(self, ctx, h, cache, residual):
        outs = []
        t = 0
        slots = cache.slots.long()
        for b, n in enumerate(ctx.new_tokens_host):
            s = cache.state[slots[b]].clone()
            for i in range(n):
                s = self.decay * s + (1 - self.decay) * h[t + i].float()
                outs.append(s)
            cache.state[slots[b]] = s
            t += n
        return self.proj.forward(torch.stack(outs).to(h.dtype))          # the block adds it to the residual


@dataclasses.dataclass(frozen=True)
class ToyConfig:
    vocab_size: int
    width: int
    n_layers: int
    decay: float
    eps: float

    @classmethod
    def from_dict(cls, raw):
        return cls(**{f.name: raw[f.name] for f in dataclasses.fields(cls)})

    def to_dict(self):
        return dict(dataclasses.asdict(self), architectures=["ToyRunningMeanLM"])


def build_toy(c: ToyConfig):
    blocks = [PreNormBlock(RMSNorm(c.width, c.eps), RunningMeanMixer(c.width, c.decay), RMSNorm(c.width, c.eps),
                           SwiGLU(c.width, 2 * c.width), names=("norm1", "mixer", "norm2", "ffn")) for _ in range(c.n_layers)]
    emb = Embedding(c.vocab_size, c.width)
    # the schedule runs layer 0 twice: a layer may be named twice and then keeps two states
    schedule = [Run(0)] + [Run(i) for i in range(c.n_layers)]
    return DecoderModel(c, emb, blocks, RMSNorm(c.width, c.eps), OutputHead(c.vocab_size, c.width, tied_to=emb),
                        schedule=schedule, names={"embedding": "tok", "blocks": "layer.{}", "final_norm": "out_norm"})


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_mixer_with_state_is_registered_built_and_stepped(tmp_path, dtype):
    wpc.register_architecture("ToyRunningMeanLM", ToyConfig, build_toy)
    try:
        cfg = ToyConfig(vocab_size=90, width=40, n_layers=2, decay=0.8, eps=1e-5)
        folder = wpc.write_random_model(str(tmp_path / "toy"), cfg, 3, getattr(torch, dtype))
        with open(os.path.join(folder, "config.json")) as f:
            assert json.load(f)["architectures"] == ["ToyRunningMeanLM"]
        eng = wpc.Engine.from_folder(folder, dtype=dtype, max_tokens=1024, max_sequences=4)
        assert len(eng.cache.groups) == 1 and eng.cache.groups[0].state.shape == (3, 4, 40)   # three scheduled runs
        toks = np.random.default_rng(0).integers(0, 90, size=30).tolist()
        from helpers import run_batch, run_tail_one_by_one, run_whole
        whole = run_whole(eng, toks)
        tail = run_tail_one_by_one(eng, toks, tail=12)       # the state carries over steps; slots are reused
        batch = run_batch(eng, [toks, toks[:11]], [20, 3])
        t = 1e-5 if dtype == "float32" else 4e-2
        scale = np.abs(whole).max()
        assert np.abs(tail - whole).max() <= t * scale
        assert np.abs(batch[0] - whole).max() <= t * scale and np.abs(batch[1] - whole[:11]).max() <= t * scale
        assert np.abs(whole[5] - whole[6]).max() > 1e-3
        out = wpc.generate(eng, [toks[:4], toks[:9]], wpc.GenerationOptions(max_tokens=5))
        assert [len(o) for o in out] == [5, 5]
        eng.cache.check()
    finally:
        wpc.unregister_architecture("ToyRunningMeanLM")


# ---- a second toy architecture: a feed-forward with routing and another position encoding -----------
from wpc_engine_b200 import ops as _ops
from wpc_engine_b200.parts import FeedForward, PositionEncoding


class RoutedFeedForward(FeedForward):
    """Each token goes to the one expert (a SwiGLU of the library) whose router logit is
    greatest; the expert's output is scaled by the softmax weight of that logit.  Router logits
    and softmax in float32.  A toy: the grouping by expert uses torch indexing, whose shapes
    depend on the data, so it cannot be captured into a graph."""
    graph_safe = False

    def __init__(self, width, inner, n_experts):
        self.width = width
        self.router = Linear(width, n_experts)
        self.experts = [SwiGLU(width, inner) for _ in range(n_experts)]

    def subparts(self):
        parts = {"router": self.router}
        parts.update({f"experts.{e}": x for e, x in enumerate(self.experts)})
        return parts

    def forward(self, ctx, h, residual):
        logits = _ops.linear(h, self.router.weight, out_dtype=torch.float32)
        prob = torch.softmax(logits.float(), dim=-1)
        top = prob.argmax(dim=-1)
        out = torch.zeros((h.shape[0], self.width), dtype=torch.float32, device=h.device)
        for e, expert in enumerate(self.experts):
            idx = (top == e).nonzero().flatten()
            if idx.numel():
                acc = torch.zeros((idx.numel(), self.width), dtype=torch.float32, device=h.device)
                expert.forward(ctx, h[idx].contiguous(), acc)          # adds its output into acc
                out[idx] = acc * prob[idx, e].unsqueeze(1)
        return out                                                       # the block adds it to the residual


class ScaledRotary(PositionEncoding):
    """Rotation by (position / factor) * theta^(-2i/head_dim): positions stretched by a factor,
    angles in float64 on the device like the library's own encoding."""

    def __init__(self, head_dim, theta, factor):
        i = np.arange(head_dim // 2, dtype=np.float64)
        self._inv = np.power(np.float64(theta), -(2.0 * i) / head_dim) / np.float64(factor)
        self._dev = None

    def tables(self, ctx):
        key = ("scaled_rotary", id(self))
        if key not in ctx.shared:
            if self._dev is None:
                self._dev = torch.from_numpy(self._inv.copy()).to(ctx.positions.device)
            ctx.shared[key] = _ops.rope_angles(ctx.positions, self._dev)
        return ctx.shared[key]


@dataclasses.dataclass(frozen=True)
class RoutedConfig:
    vocab_size: int
    width: int
    n_layers: int
    n_heads: int
    n_kv_heads: int
    inner: int
    n_experts: int
    theta: float
    factor: float
    eps: float

    @classmethod
    def from_dict(cls, raw):
        return cls(**{f.name: raw[f.name] for f in dataclasses.fields(cls)})

    def to_dict(self):
        return dict(dataclasses.asdict(self), architectures=["ToyRoutedLM"])


def build_routed(c: RoutedConfig):
    hd = c.width // c.n_heads
    pos = ScaledRotary(hd, c.theta, c.factor)                  # one object for all layers: tables are shared
    blocks = []
    for layer in range(c.n_layers):
        # odd layers route, even layers have the dense feed-forward: parts are chosen layer by layer
        ffn = RoutedFeedForward(c.width, c.inner, c.n_experts) if layer % 2 else SwiGLU(c.width, c.inner)
        blocks.append(PreNormBlock(RMSNorm(c.width, c.eps), GQAAttention(c.width, c.n_heads, c.n_kv_heads, hd, pos, qkv_bias=False),
                                   RMSNorm(c.width, c.eps), ffn, names=("ln1", "attn", "ln2", "ffn")))
    emb = Embedding(c.vocab_size, c.width)
    return DecoderModel(c, emb, blocks, RMSNorm(c.width, c.eps), OutputHead(c.vocab_size, c.width),
                        names={"embedding": "wte", "blocks": "h.{}", "final_norm": "ln_f", "head": "head"})


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_routed_feed_forward_part_alone(dtype):
    """The toy routed feed-forward against a float64 restatement: the right expert, the right weight."""
    part = RoutedFeedForward(48, 80, 3)
    ts = {"router.weight": rnd((3, 48), 61, 0.5)}
    for e in range(3):
        ts[f"experts.{e}.gate_proj.weight"] = rnd((80, 48), 62 + 3 * e, 0.1)
        ts[f"experts.{e}.up_proj.weight"] = rnd((80, 48), 63 + 3 * e, 0.1)
        ts[f"experts.{e}.down_proj.weight"] = rnd((48, 80), 64 + 3 * e, 0.1)
    ts = {k: v.to(dtype) for k, v in ts.items()}
    bind(part, ts, dtype)
    h = rnd((11, 48), 75).to(dtype)
    out = part.forward(make_ctx(dtype, [11], [0]), h.to(DEV), None).cpu().numpy()
    f = lambda t: t.float().numpy().astype(np.float64)
    logits = f(h) @ f(ts["router.weight"]).T
    prob = np.exp(logits - logits.max(-1, keepdims=True))
    prob /= prob.sum(-1, keepdims=True)
    assert len(set(prob.argmax(-1).tolist())) > 1, "the case is meant to use several experts"
    want = np.zeros((11, 48))
    for t in range(11):
        e = int(prob[t].argmax())
        want[t] = prob[t, e] * P.swiglu(f(h[t:t + 1]), f(ts[f"experts.{e}.gate_proj.weight"]),
                                        f(ts[f"experts.{e}.up_proj.weight"]), f(ts[f"experts.{e}.down_proj.weight"]))[0]
    assert np.abs(out - want).max() <= tol(dtype) * np.abs(want).max()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_routed_model_with_another_position_encoding(tmp_path, dtype):
    """Registered, built, written, loaded and stepped from here: whole prompts, the tail token by
    token, an unequal batch and generation agree, and stretching the positions changes the result."""
    wpc.register_architecture("ToyRoutedLM", RoutedConfig, build_routed)
    try:
        cfg = RoutedConfig(vocab_size=70, width=48, n_layers=3, n_heads=3, n_kv_heads=1, inner=56, n_experts=3,
                           theta=10000.0, factor=4.0, eps=1e-5)
        folder = wpc.write_random_model(str(tmp_path / "routed"), cfg, 5, getattr(torch, dtype))
        eng = wpc.Engine.from_folder(folder, dtype=dtype, max_tokens=1024, max_sequences=4)
        toks = np.random.default_rng(1).integers(0, 70, size=40).tolist()
        from helpers import run_batch, run_tail_one_by_one, run_whole
        whole = run_whole(eng, toks)
        tail = run_tail_one_by_one(eng, toks, tail=12)
        batch = run_batch(eng, [toks, toks[:13]], [25, 4])
        t = 2e-5 if dtype == "float32" else 5e-2
        scale = np.abs(whole).max()
        assert np.abs(tail - whole).max() <= t * scale
        assert np.abs(batch[0] - whole).max() <= t * scale and np.abs(batch[1] - whole[:13]).max() <= t * scale
        out = wpc.generate(eng, [toks[:4], toks[:9]], wpc.GenerationOptions(max_tokens=5))
        assert [len(o) for o in out] == [5, 5]
        eng.cache.check()
        # the same weights with unstretched positions give other logits from the second token on
        other = dataclasses.replace(cfg, factor=1.0)
        with open(os.path.join(folder, "config.json"), "w") as fjson:
            json.dump(other.to_dict(), fjson)
        eng2 = wpc.Engine.from_folder(folder, dtype=dtype, max_tokens=1024, max_sequences=4)
        whole2 = run_whole(eng2, toks)
        assert np.abs(whole2[0] - whole[0]).max() <= t * scale          # position 0 is not rotated either way
        assert np.abs(whole2[5:] - whole[5:]).max() > 1e-3 * scale
    finally:
        wpc.unregister_architecture("ToyRoutedLM")


# ---- a third toy architecture: variations of the library's own parts --------------------------------
# Attention with a norm on every head of q and k between projection and rotation (the option of
# wpc-runtime/src/model.rs:14-21, 447-462), a rotation that pairs neighbouring elements, a gated
# feed-forward with another activation, and a schedule whose second entry reads the first
# entry's keys and values instead of keeping its own.  Checked against a restatement in NumPy.
from wpc_engine_b200.parts import GatedMLP, HeadRMSNorm


class InterleavedRotary(PositionEncoding):
    """pos * theta^(-2i/head_dim) on the pairs (2i, 2i + 1)."""
    pairing = "interleaved"

    def __init__(self, head_dim, theta):
        i = np.arange(head_dim // 2, dtype=np.float64)
        self._inv = np.power(np.float64(theta), -(2.0 * i) / head_dim)
        self._dev = None

    def tables(self, ctx):
        key = ("interleaved_rotary", id(self))
        if key not in ctx.shared:
            if self._dev is None:
                self._dev = torch.from_numpy(self._inv.copy()).to(ctx.positions.device)
            ctx.shared[key] = _ops.rope_angles(ctx.positions, self._dev)
        return ctx.shared[key]


@dataclasses.dataclass(frozen=True)
class VariantConfig:
    vocab_size: int
    width: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    inner: int
    theta: float
    eps: float
    longest: int

    @classmethod
    def from_dict(cls, raw):
        return cls(**{f.name: raw[f.name] for f in dataclasses.fields(cls)})

    def to_dict(self):
        return dict(dataclasses.asdict(self), architectures=["ToyVariantLM"])


VARIANT_SCHEDULE = [(0, None), (1, 0), (2, None)]        # (layer, the schedule entry whose cache it reads)


def build_variant(c: VariantConfig):
    pos = InterleavedRotary(c.head_dim, c.theta)
    blocks = []
    for _ in range(3):
        attn = GQAAttention(c.width, c.n_heads, c.n_kv_heads, c.head_dim, pos, qkv_bias=False,
                            q_norm=HeadRMSNorm(c.head_dim, c.eps), k_norm=HeadRMSNorm(c.head_dim, c.eps))
        blocks.append(PreNormBlock(RMSNorm(c.width, c.eps), attn, RMSNorm(c.width, c.eps),
                                   GatedMLP(c.width, c.inner, "gelu_tanh"), names=("ln1", "attn", "ln2", "ffn")))
    emb = Embedding(c.vocab_size, c.width)
    return DecoderModel(c, emb, blocks, RMSNorm(c.width, c.eps), OutputHead(c.vocab_size, c.width),
                        schedule=[Run(layer, cache_of=src) for layer, src in VARIANT_SCHEDULE],
                        names={"embedding": "wte", "blocks": "h.{}", "final_norm": "ln_f", "head": "head"},
                        max_positions=c.longest)


def variant_plain(c: VariantConfig, tensors, tokens):
    """The toy model for a whole sequence in float64, from the formulas alone."""
    w = {k: v.astype(np.float64) for k, v in tensors.items()}
    T = len(tokens)
    hd, half = c.head_dim, c.head_dim // 2
    inv = np.power(np.float64(c.theta), -(2.0 * np.arange(half)) / hd)
    ang = np.arange(T, dtype=np.float64)[:, None] * inv[None, :]
    cs, sn = np.cos(ang).astype(np.float32).astype(np.float64), np.sin(ang).astype(np.float32).astype(np.float64)

    def rotate(v):                                    # [T, heads, hd], pairs (2i, 2i + 1)
        out = v.copy()
        a, b = v[..., 0::2], v[..., 1::2]
        out[..., 0::2] = a * cs[:, None, :] - b * sn[:, None, :]
        out[..., 1::2] = b * cs[:, None, :] + a * sn[:, None, :]
        return out

    x = w["wte.weight"][np.asarray(tokens)]
    kept = {}
    for i, (layer, src) in enumerate(VARIANT_SCHEDULE):
        p = f"h.{layer}"
        n1 = P.rms_norm(x, w[f"{p}.ln1.weight"], c.eps)
        q = (n1 @ w[f"{p}.attn.q_proj.weight"].T).reshape(T, c.n_heads, hd)
        q = rotate(P.rms_norm(q, w[f"{p}.attn.q_norm.weight"], c.eps))
        if src is None:
            k = (n1 @ w[f"{p}.attn.k_proj.weight"].T).reshape(T, c.n_kv_heads, hd)
            k = rotate(P.rms_norm(k, w[f"{p}.attn.k_norm.weight"], c.eps))
            v = (n1 @ w[f"{p}.attn.v_proj.weight"].T).reshape(T, c.n_kv_heads, hd)
            kept[i] = (k, v)
        else:
            k, v = kept[src]
        x = x + P.attention(q, k, v).reshape(T, -1) @ w[f"{p}.attn.o_proj.weight"].T
        n2 = P.rms_norm(x, w[f"{p}.ln2.weight"], c.eps)
        g, u = n2 @ w[f"{p}.ffn.gate_proj.weight"].T, n2 @ w[f"{p}.ffn.up_proj.weight"].T
        act = 0.5 * g * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (g + 0.044715 * g ** 3)))
        x = x + (act * u) @ w[f"{p}.ffn.down_proj.weight"].T
    return P.rms_norm(x, w["ln_f.weight"], c.eps) @ w["head.weight"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("sizes", [dict(width=48, n_heads=3, n_kv_heads=1, head_dim=16, inner=56),
                                   dict(width=256, n_heads=4, n_kv_heads=2, head_dim=64, inner=384)])
def test_toy_model_of_varied_parts_against_numpy(tmp_path, dtype, sizes):
    """Head norms, interleaved pairs, another activation, a layer that reads another layer's
    cache: whole, tail one by one and in an unequal batch against the NumPy restatement."""
    wpc.register_architecture("ToyVariantLM", VariantConfig, build_variant)
    try:
        cfg = VariantConfig(vocab_size=150, theta=10000.0, eps=1e-5, longest=256, **sizes)
        folder = wpc.write_random_model(str(tmp_path / "variant"), cfg, 9, getattr(torch, dtype))
        eng = wpc.Engine.from_folder(folder, dtype=dtype, max_tokens=2048, max_sequences=4)
        assert eng.max_positions == 256 and eng.vocab_size == 150
        # three schedule entries, two of them with a cache of their own
        assert eng.model.cache_specs()[1] is None and eng.cache.groups[0].n_layers == 2
        _, tensors = P.read_model_folder(folder)
        toks = np.random.default_rng(2).integers(0, 150, size=90).tolist()
        want = variant_plain(cfg, tensors, toks)
        from helpers import bfloat16_bound, run_batch, run_tail_one_by_one, run_whole
        bound = 2e-4 * np.abs(want).max() if dtype == "float32" else bfloat16_bound(want)
        assert np.abs(run_whole(eng, toks) - want).max() <= bound
        assert np.abs(run_tail_one_by_one(eng, toks, tail=30) - want).max() <= bound
        batch = run_batch(eng, [toks, toks[:21]], [70, 5])
        assert np.abs(batch[0] - want).max() <= bound and np.abs(batch[1] - want[:21]).max() <= bound
        # the parts matter: without the head norms the logits are others
        for b in eng.model.blocks:
            b.mixer.q_norm = b.mixer.k_norm = None
        assert np.abs(run_whole(eng, toks) - want).max() > 10 * bound
        slot = eng.open_sequence()
        with pytest.raises(ValueError, match="longest sequence"):
            eng.step([SequenceStep(slot, [1] * 257, want=[])])
        eng.close_sequence(slot)
        eng.cache.check()
    finally:
        wpc.unregister_architecture("ToyVariantLM")
