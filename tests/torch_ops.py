"""Plain torch restatements of the device operations, one function per kernel, with the same
signatures as wpc_engine_b200/ops.py.  They serve the tests in two ways: as the plain
reference that each kernel is compared with on the GPU, and (patched in by the `cpu_ops`
fixture) as stand-ins that let the engine's host logic run on a machine without a GPU.
Arithmetic is float32 (float64 for the rotation angles), results are rounded once to the
output type.  Formulas: wpc-runtime/src/norm.rs:4-13, rope.rs:24-40, model.rs:476-531,
sampling.rs:3-51."""
import math

import torch

PAGE = 64
__all__ = ["require_device", "embed", "rmsnorm", "linear", "silu_mul", "gate_mul", "gated_linear", "add_", "gather_rows",
           "convert", "rope_angles", "rope_inplace", "head_rmsnorm_", "qk_rope_kv_store", "linear_qk_rope_kv_store",
           "attention", "sample", "fill_normal"]

_M64 = (1 << 64) - 1


def require_device(device="cuda"):
    return None


def embed(tokens, table):
    return table[tokens.long()].float()


def rmsnorm(x, gain, eps, out_dtype, rows=None):
    if rows is not None:
        x = x[rows.long()]
    ms = (x * x).sum(-1, keepdim=True) / x.shape[-1]
    return (x * (1.0 / torch.sqrt(ms + eps)) * gain).to(out_dtype)


def linear(x, w, bias=None, out_dtype=None, residual=None, plain=False, static_weight=False):
    y = x.float() @ w.float().t()
    if bias is not None:
        y = y + bias
    if residual is not None:
        residual += y
        return residual
    return y.to(out_dtype or x.dtype)


GATED_GROUP = 64


def activation(name, g):
    if name == "silu":
        return g / (1.0 + torch.exp(-g))
    if name == "gelu_tanh":
        return 0.5 * g * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (g + 0.044715 * g * g * g)))
    raise ValueError(name)


def gate_mul(gu, inner, group=None, activation_name="silu"):
    group = inner if group is None else group
    v = gu.float().reshape(gu.shape[0], inner // group, 2, group)
    g, u = v[:, :, 0].reshape(gu.shape[0], inner), v[:, :, 1].reshape(gu.shape[0], inner)
    return (activation(activation_name, g) * u).to(gu.dtype)


def silu_mul(gu, inner, group=None):
    return gate_mul(gu, inner, group, "silu")


def gated_linear(x, w, inner, group, plain=False, static_weight=False, activation="silu"):
    return gate_mul(linear(x, w), inner, group, activation)


def add_(x, y):
    x += y.float()
    return x


def gather_rows(x, idx):
    return x[idx.long()].clone()


def convert(x, dtype):
    return x.to(dtype)


def rope_angles(positions, inv_freq):
    a = positions.double()[:, None] * inv_freq[None, :]
    return torch.cos(a).float(), torch.sin(a).float()


def _rotate(v, cos, sin, head_dim, interleaved=False):
    # v: [T, heads, head_dim] float32
    half, R = head_dim // 2, cos.shape[1]
    out = v.clone()
    c, s = cos[:, None, :], sin[:, None, :]
    if interleaved:
        x1, x2 = v[..., 0:2 * R:2], v[..., 1:2 * R:2]
        out[..., 0:2 * R:2] = x1 * c - x2 * s
        out[..., 1:2 * R:2] = x2 * c + x1 * s
        return out
    x1, x2 = v[..., :R], v[..., half:half + R]
    out[..., :R] = x1 * c - x2 * s
    out[..., half:half + R] = x2 * c + x1 * s
    return out


def rope_inplace(x, n_heads, head_dim, cos, sin, interleaved=False):
    T = x.shape[0]
    v = x[:, :n_heads * head_dim].float().reshape(T, n_heads, head_dim)
    x[:, :n_heads * head_dim] = _rotate(v, cos, sin, head_dim, interleaved).reshape(T, -1).to(x.dtype)
    return x


def head_rmsnorm_(x, n_heads, head_dim, gain, eps):
    T = x.shape[0]
    v = x[:, :n_heads * head_dim].float().reshape(T, n_heads, head_dim)
    ms = (v * v).sum(-1, keepdim=True) / head_dim
    x[:, :n_heads * head_dim] = (v * (1.0 / torch.sqrt(ms + eps)) * gain).reshape(T, -1).to(x.dtype)
    return x


def qk_rope_kv_store(qkv, n_heads, n_kv_heads, head_dim, cos, sin, k_pages, v_pages, page_table,
                     seq_of_token, positions):
    T = qkv.shape[0]
    nq, nk = n_heads * head_dim, n_kv_heads * head_dim
    k = qkv[:, nq:nq + nk].float().reshape(T, n_kv_heads, head_dim)
    if cos is not None:
        rope_inplace(qkv, n_heads, head_dim, cos, sin)
        k = _rotate(k, cos, sin, head_dim)
    v = qkv[:, nq + nk:].reshape(T, n_kv_heads, head_dim)
    for t in range(T):
        pos, b = int(positions[t]), int(seq_of_token[t])
        page = int(page_table[b, pos // PAGE])
        assert page >= 0
        k_pages[page, :, pos % PAGE, :] = k[t].to(k_pages.dtype)
        v_pages[page, :, pos % PAGE, :] = v[t]


def linear_qk_rope_kv_store(x, w, bias, n_heads, n_kv_heads, head_dim, cos, sin, k_pages, v_pages, page_table,
                            seq_of_token, positions):
    qkv = linear(x, w, bias)
    qk_rope_kv_store(qkv, n_heads, n_kv_heads, head_dim, cos, sin, k_pages, v_pages, page_table, seq_of_token, positions)
    return qkv


def attention(q, n_heads, n_kv_heads, head_dim, k_pages, v_pages, page_table, cu_seqlens, ctx_lens,
              seq_of_token, positions, scale, window, max_new_tokens, max_ctx_len, splits=None, mma_only=False,
              cluster=None, groups=1):
    return attention_plain(q, n_heads, n_kv_heads, head_dim, k_pages, v_pages, page_table, seq_of_token,
                           positions, scale, window)


def attention_plain(q, n_heads, n_kv_heads, head_dim, k_pages, v_pages, page_table, seq_of_token, positions,
                    scale, window, max_ctx_len=None, splits=None):
    T = q.shape[0]
    out = torch.zeros((T, n_heads * head_dim), dtype=torch.float32, device=q.device)
    n_rep = n_heads // n_kv_heads
    for t in range(T):
        pos, b = int(positions[t]), int(seq_of_token[t])
        lo = max(0, pos - window + 1) if window else 0
        idx = torch.arange(lo, pos + 1, device=q.device)
        pages = page_table[b, (idx // PAGE).long()].long()
        assert int(pages.min()) >= 0
        k = k_pages[pages, :, (idx % PAGE).long(), :].float()       # [n, nkv, hd]
        v = v_pages[pages, :, (idx % PAGE).long(), :].float()
        for h in range(n_heads):
            qv = q[t, h * head_dim:(h + 1) * head_dim].float()
            s = (k[:, h // n_rep, :] @ qv) * scale
            p = torch.softmax(s, dim=0)
            out[t, h * head_dim:(h + 1) * head_dim] = p @ v[:, h // n_rep, :]
    return out.to(q.dtype)


def _mix64(z):
    z = (z + 0x9E3779B97F4A7C15) & _M64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M64
    return z ^ (z >> 31)


def sample(logits, slots, seq_state, temperature, banned):
    out = []
    ban = set(banned.tolist()) if banned is not None else set()
    for row in range(logits.shape[0]):
        z = logits[row].double().clone()
        for b in ban:
            z[b] = -math.inf
        st = seq_state[int(slots[row])]
        if not temperature > 0 or bool(torch.isinf(z).all()):
            best, best_v = 0, -math.inf
            for i, v in enumerate(z.tolist()):
                if v > best_v:
                    best, best_v = i, v
            out.append(best)
        else:
            r = _mix64(int(st[1]) & _M64)
            r = _mix64(r ^ (int(st[2]) & _M64))
            r = _mix64(r ^ (int(st[3]) & _M64))
            u = (r >> 40) / float(1 << 24)
            e = torch.exp((z - z.max()) / temperature)
            cdf = torch.cumsum(e, 0)
            idx = int(torch.searchsorted(cdf, torch.tensor(u * float(cdf[-1]), dtype=cdf.dtype), right=True))
            out.append(min(idx, z.numel() - 1))
        st[3] += 1
    return torch.tensor(out, dtype=torch.int32, device=logits.device)


def fill_normal(t, key, mean, std):
    g = torch.Generator().manual_seed(key & ((1 << 62) - 1))
    t.copy_((torch.randn(t.shape, generator=g) * std + mean).to(t.dtype))
