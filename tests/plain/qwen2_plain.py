"""Plain, slow implementation of the Qwen2 dense decoder, used only by the tests.

It rests on the formulas of the reference (jpytka666-jpg/wpc-engine), restated in NumPy; the
reference is a Rust workspace and no Rust toolchain exists here, so it could not be compiled or
run for a numeric comparison.  The anchor vectors of the reference's own unit tests
(wpc-runtime/src/norm.rs:49-89, rope.rs:46-72, sampling.rs:57-74) are replayed against these
functions in tests/test_plain.py instead.

Whole sequences, no cache, one function for each part.  Nothing here is imported by the
package and nothing of the package is imported here: file reading, weight naming and the
arithmetic are all restated.  `dtype` selects float32 (the reference's precision) or float64
(the yardstick that both the reference precision and the GPU paths are measured against).
"""
from __future__ import annotations

import json
import math
import os
import struct

import numpy as np


# ---------------------------------------------------------------------------------------------
# model folder reading (own reader: the format is an 8-byte little-endian header length, a JSON
# header with dtype/shape/data_offsets per tensor, then the raw bytes)
# ---------------------------------------------------------------------------------------------
def read_model_folder(folder):
    """Returns (config dict, {tensor name: float32 ndarray}).

    Decoding follows wpc-runtime/src/weights.rs:149-176: F32 as is, F16 widened, BF16 as
    `bits << 16`; anything else is an error.
    """
    with open(os.path.join(folder, "config.json")) as f:
        config = json.load(f)
    path = os.path.join(folder, "model.safetensors")
    with open(path, "rb") as f:
        (hlen,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(hlen).decode("utf-8"))
        blob = f.read()
    tensors = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        lo, hi = meta["data_offsets"]
        raw = blob[lo:hi]
        if meta["dtype"] == "F32":
            arr = np.frombuffer(raw, dtype="<f4").astype(np.float32)
        elif meta["dtype"] == "F16":
            arr = np.frombuffer(raw, dtype="<f2").astype(np.float32)
        elif meta["dtype"] == "BF16":
            bits = np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16
            arr = bits.view(np.float32)
        else:
            raise ValueError(f"tensor {name}: unsupported dtype {meta['dtype']}")
        tensors[name] = arr.reshape(meta["shape"])
    return config, tensors


def head_dim_of(config):
    """wpc-runtime/src/config.rs:59-62: the stated head_dim, else hidden_size / heads."""
    hd = config.get("head_dim")
    return hd if hd is not None else config["hidden_size"] // config["num_attention_heads"]


# ---------------------------------------------------------------------------------------------
# the parts
# ---------------------------------------------------------------------------------------------
def rms_norm(x, weight, eps):
    """wpc-runtime/src/norm.rs:4-13: mean of squares, 1/sqrt(ms + eps), then x * scale * w.

    x: [..., n]; statistics over the last axis, in x's dtype.
    """
    dt = x.dtype
    n = dt.type(x.shape[-1])
    mean_sq = np.sum(x * x, axis=-1, keepdims=True, dtype=dt) / n
    scale = dt.type(1.0) / np.sqrt(mean_sq + dt.type(eps))
    return x * scale * weight.astype(dt)


def softmax(x):
    """wpc-runtime/src/norm.rs:28-43: subtract the maximum, exponentiate, divide by the sum."""
    m = np.max(x, axis=-1, keepdims=True)
    e = np.exp(x - m)
    s = np.sum(e, axis=-1, keepdims=True, dtype=x.dtype)
    return np.where(s > 0, e / np.where(s > 0, s, 1), e)


def rope(x, positions, theta):
    """wpc-runtime/src/rope.rs:24-40 with rotary_pairs = d/2 (rope.rs:10-13).

    x: [T, heads, d]; positions: [T] integers.  Angles, sine and cosine are computed in
    float64 and cast to x's dtype, pairs are (i, i + d/2).
    """
    T, _, d = x.shape
    half = d // 2
    i = np.arange(half, dtype=np.float64)
    inv_freq = np.power(np.float64(theta), -(2.0 * i) / np.float64(d))
    angle = np.asarray(positions, dtype=np.float64)[:, None] * inv_freq[None, :]
    s = np.sin(angle).astype(x.dtype)[:, None, :]
    c = np.cos(angle).astype(x.dtype)[:, None, :]
    x1 = x[..., :half]
    x2 = x[..., half:]
    out = np.empty_like(x)
    out[..., :half] = x1 * c - x2 * s
    out[..., half:] = x2 * c + x1 * s
    return out


def linear(x, weight, bias=None):
    """wpc-runtime/src/weights.rs:59-78: y = W x (+ b), W is [out, in] row-major."""
    y = x @ weight.astype(x.dtype, copy=False).T
    if bias is not None:
        y = y + bias.astype(x.dtype, copy=False)
    return y


def attention(q, k, v, window=None):
    """wpc-runtime/src/model.rs:476-510 for every position of one whole sequence.

    q: [T, nh, d] (rotated), k: [T, nkv, d] (rotated), v: [T, nkv, d].  Query head qh reads
    KV head qh // n_rep (model.rs:484); scores are scaled by 1/sqrt(d) (model.rs:477); the
    query at position p sees positions 0..p (the cache holds nothing later, model.rs:476).
    `window` (not in the reference, which ignores the key; config.rs:162-168): when given,
    the query at p sees only the last `window` positions p-window+1..p.
    """
    T, nh, d = q.shape
    nkv = k.shape[1]
    n_rep = nh // nkv
    dt = q.dtype
    scale = dt.type(1.0) / np.sqrt(dt.type(d))
    out = np.zeros((T, nh, d), dtype=dt)
    pos = np.arange(T)
    visible = pos[None, :] <= pos[:, None]
    if window is not None:
        visible &= pos[None, :] > pos[:, None] - window
    for qh in range(nh):
        kvh = qh // n_rep
        scores = (q[:, qh, :] @ k[:, kvh, :].T) * scale
        scores = np.where(visible, scores, dt.type(-np.inf))
        p = softmax(scores)
        out[:, qh, :] = p @ v[:, kvh, :]
    return out


def swiglu(x, w_gate, w_up, w_down):
    """wpc-runtime/src/model.rs:518-536: down( gate/(1+exp(-gate)) * up ), no biases."""
    g = linear(x, w_gate)
    u = linear(x, w_up)
    act = g / (x.dtype.type(1.0) + np.exp(-g)) * u
    return linear(act, w_down)


def layer_uses_window(config, layer):
    """Not in the reference.  The config keys' own meaning: with use_sliding_window set, the
    first max_window_layers layers attend to everything and the later ones to a window."""
    if not config.get("use_sliding_window", False) or config.get("sliding_window") is None:
        return False
    return layer >= config.get("max_window_layers", 0)


class _Converted:
    """tensors[name] in another dtype, converted when it is asked for (a model of real size
    would not fit twice in memory)."""

    def __init__(self, tensors, dt):
        self.tensors, self.dt = tensors, dt

    def __getitem__(self, name):
        return self.tensors[name].astype(self.dt, copy=False)


def forward(config, tensors, tokens, dtype=np.float32, rows=None):
    """wpc-runtime/src/model.rs:419-547 for a whole sequence: logits [T, vocab] in `dtype`.

    Row t holds the logits for the token after position t.  The output head is the
    embedding table when tie_word_embeddings is true (its default, config.rs:18-19;
    model.rs:544-546 always takes that branch) and `lm_head.weight` when it is false.
    `rows`: the positions whose logits are computed (all by default); the layers always run
    on the whole sequence.
    """
    dt = np.dtype(dtype)
    w = _Converted(tensors, dt)
    nh = config["num_attention_heads"]
    nkv = config["num_key_value_heads"]
    hd = head_dim_of(config)
    eps = config["rms_norm_eps"]
    theta = config["rope_theta"]
    tokens = np.asarray(tokens, dtype=np.int64)
    T = tokens.shape[0]
    positions = np.arange(T)

    x = tensors["model.embed_tokens.weight"][tokens].astype(dt)     # model.rs:429-430
    for l in range(config["num_hidden_layers"]):
        p = f"model.layers.{l}"
        n1 = rms_norm(x, w[f"{p}.input_layernorm.weight"], eps)     # model.rs:434-435
        q = linear(n1, w[f"{p}.self_attn.q_proj.weight"], w[f"{p}.self_attn.q_proj.bias"])
        k = linear(n1, w[f"{p}.self_attn.k_proj.weight"], w[f"{p}.self_attn.k_proj.bias"])
        v = linear(n1, w[f"{p}.self_attn.v_proj.weight"], w[f"{p}.self_attn.v_proj.bias"])
        q = rope(q.reshape(T, nh, hd), positions, theta)            # model.rs:464-469
        k = rope(k.reshape(T, nkv, hd), positions, theta)
        v = v.reshape(T, nkv, hd)
        window = config["sliding_window"] if layer_uses_window(config, l) else None
        a = attention(q, k, v, window).reshape(T, nh * hd)
        x = x + linear(a, w[f"{p}.self_attn.o_proj.weight"])        # model.rs:512-516
        n2 = rms_norm(x, w[f"{p}.post_attention_layernorm.weight"], eps)
        x = x + swiglu(n2, w[f"{p}.mlp.gate_proj.weight"], w[f"{p}.mlp.up_proj.weight"],
                       w[f"{p}.mlp.down_proj.weight"])              # model.rs:518-536
    if rows is not None:
        x = x[np.asarray(rows, dtype=np.int64)]
    xf = rms_norm(x, w["model.norm.weight"], eps)                   # model.rs:541-542
    tied = config.get("tie_word_embeddings", True)
    head = w["model.embed_tokens.weight"] if tied else w["lm_head.weight"]
    return linear(xf, head)                                          # model.rs:544-546


# ---------------------------------------------------------------------------------------------
# sampling and generation
# ---------------------------------------------------------------------------------------------
def argmax(logits, banned=()):
    """wpc-runtime/src/sampling.rs:3-13 and 35-51: the first strictly greatest value wins,
    banned ids are skipped, NaN never wins, an empty or all-banned input gives 0."""
    best_i, best_v = 0, -math.inf
    banned = set(int(b) for b in banned)
    for i, v in enumerate(np.asarray(logits).tolist()):
        if i in banned:
            continue
        if v > best_v:
            best_v, best_i = v, i
    return best_i


_M64 = (1 << 64) - 1


def _mix64(z):
    z = (z + 0x9E3779B97F4A7C15) & _M64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M64
    return z ^ (z >> 31)


def uniform_for(seed, request, step):
    """The uniform number in [0, 1) that the sampler of this library draws for the `step`-th
    generated token of request number `request` under `seed` (not in the reference, which
    has no random sampling): three rounds of the splitmix64 finalizer, top 24 bits."""
    z = _mix64(seed & _M64)
    z = _mix64(z ^ (request & _M64))
    z = _mix64(z ^ (step & _M64))
    return (z >> 40) * (1.0 / (1 << 24))


def sample_temperature(logits, temperature, u, banned=()):
    """Not in the reference.  p = softmax(logits / temperature); returns the first index
    whose cumulative probability exceeds u * sum(p), and the float64 cumulative sums."""
    z = np.asarray(logits, dtype=np.float64) / float(temperature)
    for b in banned:
        z[int(b)] = -np.inf
    e = np.exp(z - np.max(z))
    cdf = np.cumsum(e)
    target = u * cdf[-1]
    idx = int(np.searchsorted(cdf, target, side="right"))
    return min(idx, len(cdf) - 1), cdf, target


def generate_greedy(config, tensors, prompt, max_tokens, stop_ids=(), dtype=np.float32):
    """wpc-runtime/src/main.rs:284-312: pick, append, stop if it is a stop id (the stop id
    stays in the output and is not fed), else feed it.  Recomputes the whole sequence for
    every token; only for tiny models."""
    seq = list(prompt)
    out = []
    for _ in range(max_tokens):
        logits = forward(config, tensors, seq, dtype)[-1]
        nxt = argmax(logits)
        out.append(nxt)
        if nxt in stop_ids:
            break
        seq.append(nxt)
    return out
