"""Each kernel alone against its plain torch reference (tests/torch_ops.py), at sizes other
than the engine's: widths that are no power of two, head sizes in steps of 16, odd counts."""
import math

import numpy as np
import pytest
import torch

import torch_ops as ref
from wpc_engine_b200 import ops

pytestmark = pytest.mark.gpu
DEV = "cuda"
DTYPES = [torch.float32, torch.bfloat16]


def rnd(shape, dtype=torch.float32, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype).to(DEV)


def close(got, want, dtype, scale=1.0):
    tol = 2e-5 if dtype == torch.float32 else 1.2e-2
    err = (got.float() - want.float()).abs().max().item()
    ref_mag = max(want.float().abs().max().item(), 1e-6)
    assert err <= tol * max(ref_mag, scale), f"max error {err} against magnitude {ref_mag}"


@pytest.mark.parametrize("dtype", DTYPES)
def test_embed(dtype):
    table = rnd((301, 72), dtype, 1)
    tokens = torch.tensor([0, 300, 7, 7, 150], dtype=torch.int32, device=DEV)
    assert torch.equal(ops.embed(tokens, table), ref.embed(tokens, table))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [4, 72, 1000, 3584, 18001])
def test_rmsnorm(dtype, width):
    x = rnd((5, width), seed=2, scale=3.0)
    gain = 1 + rnd((width,), seed=3, scale=0.1)
    close(ops.rmsnorm(x, gain, 1e-5, dtype), ref.rmsnorm(x, gain, 1e-5, dtype), dtype)
    # the rows whose logits are wanted, gathered and normed in one kernel
    rows = torch.tensor([4, 0, 4, 2], dtype=torch.int32, device=DEV)
    got = ops.rmsnorm(x, gain, 1e-5, dtype, rows=rows)
    assert got.shape == (4, width) and torch.equal(got, ops.rmsnorm(x, gain, 1e-5, dtype)[rows.long()])


def test_rmsnorm_anchor():
    # wpc-runtime/src/norm.rs:49-60
    x = torch.tensor([[3.0, 4.0, 0.0, 0.0]], device=DEV)
    out = ops.rmsnorm(x, torch.ones(4, device=DEV), 1e-6, torch.float32)
    want = x.cpu() / math.sqrt(6.25 + 1e-6)
    assert torch.allclose(out.cpu(), want, atol=1e-6)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(1, 40, 24), (7, 200, 96), (130, 72, 200), (33, 300, 80)])
@pytest.mark.parametrize("mode", ["plain", "bias", "residual"])
def test_linear(dtype, shape, mode):
    M, N, K = shape
    x, w = rnd((M, K), dtype, 4), rnd((N, K), dtype, 5, 0.1)
    bias = rnd((N,), seed=6) if mode != "plain" else None
    if mode == "residual":
        r0 = rnd((M, N), seed=7)
        got = ops.linear(x, w, bias, residual=r0.clone())
        want = ref.linear(x, w, bias, residual=r0.clone())
        close(got, want, torch.float32, scale=1.0)
    else:
        close(ops.linear(x, w, bias), ref.linear(x, w, bias), dtype)


@pytest.mark.parametrize("M", [1, 2, 3, 5, 8, 9, 16, 17])
@pytest.mark.parametrize("N,K", [(40, 24), (33, 1030), (130, 2056), (1000, 520), (7, 4100)])
@pytest.mark.parametrize("dtypes", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16),
                                    (torch.float32, torch.bfloat16), (torch.bfloat16, torch.float32)])
def test_plain_linear_of_few_rows(M, N, K, dtypes):
    """The float32 product for up to 16 rows streams the weights once (every count of rows on both
    sides of 16, widths that are no multiples of 4 or of the chunk, rows that start unaligned),
    with bias, into float32 or bfloat16 or added to a residual: against float64."""
    xd, wd = dtypes
    x, w = rnd((M, K + 3), xd, 14)[:, 3:], rnd((N, K), wd, 15, 0.1)          # x: a view whose rows are unaligned
    bias = rnd((N,), seed=16)
    want = (x.double().cpu() @ w.double().cpu().t() + bias.double().cpu())
    mag = want.abs().max().item()
    got = ops.linear_plain(x, w, bias, out_dtype=torch.float32)
    assert (got.double().cpu() - want).abs().max().item() <= 3e-6 * mag * max(1.0, (K / 1000) ** 0.5)
    xc = torch.empty((M, K), dtype=xd, device=DEV).copy_(x)          # the same rows, aligned
    got16 = ops.linear_plain(xc, w, bias, out_dtype=torch.bfloat16)
    assert (got16.double().cpu() - want).abs().max().item() <= 1e-2 * mag
    r0 = rnd((M, N), seed=17)
    acc = ops.linear_plain(xc, w, None, residual=r0.clone())
    assert (acc.double().cpu() - (want - bias.double().cpu() + r0.double().cpu())).abs().max().item() <= 1e-5 * max(mag, 1.0)
    # a row's result does not depend on the rows beside it (the same kernel and the same alignment)
    alone = ops.linear_plain(xc[:1].clone(), w, bias, out_dtype=torch.float32)
    if M <= 16:
        assert torch.equal(alone[0], ops.linear_plain(xc, w, bias, out_dtype=torch.float32)[0])


def test_linear_keeps_32_bit_weights_with_16_bit_rows():
    x, w = rnd((9, 48), torch.bfloat16, 8), rnd((20, 48), torch.float32, 9)
    close(ops.linear(x, w), ref.linear(x, w), torch.bfloat16)


@pytest.mark.parametrize("dtype", DTYPES)
def test_silu_mul_add_gather_convert(dtype):
    gu = rnd((6, 2 * 77), dtype, 10, 2.0)
    close(ops.silu_mul(gu, 77), ref.silu_mul(gu, 77), dtype)
    x, y = rnd((6, 77), seed=11), rnd((6, 77), dtype, 12)
    close(ops.add_(x.clone(), y), ref.add_(x.clone(), y), torch.float32)
    idx = torch.tensor([5, 0, 5], dtype=torch.int32, device=DEV)
    assert torch.equal(ops.gather_rows(x, idx), x[idx.long()])
    assert torch.equal(ops.convert(x, torch.bfloat16), x.to(torch.bfloat16))


def test_rope_angles_and_anchor():
    # float64 angles; position 0 is the identity, pair norms are kept (wpc-runtime/src/rope.rs:46-72)
    hd, theta = 48, 1e6
    inv = torch.tensor(np.power(theta, -2.0 * np.arange(hd // 2) / hd), dtype=torch.float64, device=DEV)
    pos = torch.tensor([0, 5, 1000, 131071], dtype=torch.int32, device=DEV)
    cos, sin = ops.rope_angles(pos, inv)
    rc, rs = ref.rope_angles(pos.cpu(), inv.cpu())
    assert (cos.cpu() - rc).abs().max() <= 1e-7 and (sin.cpu() - rs).abs().max() <= 1e-7
    x = rnd((4, 3 * hd), seed=13)
    y = ops.rope_inplace(x.clone(), 3, hd, cos, sin)
    assert torch.equal(y[0], x[0])
    xv, yv = x.view(4, 3, 2, hd // 2), y.view(4, 3, 2, hd // 2)
    assert torch.allclose((xv ** 2).sum(2), (yv ** 2).sum(2), rtol=1e-5)
    close(y, ref.rope_inplace(x.clone(), 3, hd, cos, sin), torch.float32)


def paged_case(dtype, nh, nkv, hd, lens, new, window=None, seed=0):
    """A batch of sequences with `lens[b]` positions after the step, the last `new[b]` of which
    are this step's tokens; pages are handed out in a scrambled order."""
    B = len(lens)
    width = max((n + 63) // 64 for n in lens) + 1
    n_pages = sum((n + 63) // 64 for n in lens) + 3
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(seed)).tolist()
    table = torch.full((B, width), -1, dtype=torch.int32)
    for b, n in enumerate(lens):
        for i in range((n + 63) // 64):
            table[b, i] = perm.pop()
    T = sum(new)
    seq = torch.tensor([b for b in range(B) for _ in range(new[b])], dtype=torch.int32)
    pos = torch.tensor([lens[b] - new[b] + i for b in range(B) for i in range(new[b])], dtype=torch.int32)
    k_pages = rnd((n_pages, nkv, 64, hd), dtype, seed + 1)
    v_pages = rnd((n_pages, nkv, 64, hd), dtype, seed + 2)
    qkv = rnd((T, (nh + 2 * nkv) * hd), dtype, seed + 3)
    return qkv, k_pages, v_pages, table.to(DEV), seq.to(DEV), pos.to(DEV)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,hd", [(4, 2, 16), (3, 1, 32), (6, 3, 48), (7, 1, 128), (2, 2, 80)])
def test_qk_rope_kv_store(dtype, nh, nkv, hd):
    lens, new = [70, 5, 130], [6, 5, 1]
    qkv, kp, vp, table, seq, pos = paged_case(dtype, nh, nkv, hd, lens, new)
    inv = torch.tensor(np.power(1e4, -2.0 * np.arange(hd // 2) / hd), dtype=torch.float64, device=DEV)
    cos, sin = ops.rope_angles(pos, inv)
    q1, k1, v1 = qkv.clone(), kp.clone(), vp.clone()
    ops.qk_rope_kv_store(q1, nh, nkv, hd, cos, sin, k1, v1, table, seq, pos)
    q2, k2, v2 = qkv.cpu().clone(), kp.cpu().clone(), vp.cpu().clone()
    ref.qk_rope_kv_store(q2, nh, nkv, hd, cos.cpu(), sin.cpu(), k2, v2, table.cpu(), seq.cpu(), pos.cpu())
    close(q1[:, :nh * hd].cpu(), q2[:, :nh * hd], dtype)
    close(k1.cpu(), k2, dtype)
    assert torch.equal(v1.cpu(), v2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,hd", [(4, 2, 16), (3, 1, 32), (6, 3, 48), (7, 1, 128), (28, 4, 128), (2, 2, 80)])
@pytest.mark.parametrize("window", [None, 40])
def test_attention(dtype, nh, nkv, hd, window):
    lens, new = [200, 5, 131, 64], [37, 5, 1, 1]
    qkv, kp, vp, table, seq, pos = paged_case(dtype, nh, nkv, hd, lens, new, seed=5)
    cu = torch.tensor(np.concatenate([[0], np.cumsum(new)]), dtype=torch.int32, device=DEV)
    ctx = torch.tensor(lens, dtype=torch.int32, device=DEV)
    scale = 1.0 / math.sqrt(hd)
    got = ops.attention(qkv, nh, nkv, hd, kp, vp, table, cu, ctx, seq, pos, scale, window, max(new), max(lens))
    want = ref.attention_plain(qkv.cpu(), nh, nkv, hd, kp.cpu(), vp.cpu(), table.cpu(), seq.cpu(), pos.cpu(),
                               scale, window)
    close(got.cpu(), want, dtype)
    plain = ops.attention_plain(qkv, nh, nkv, hd, kp, vp, table, seq, pos, scale, window)
    close(plain.cpu(), want, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("splits", [2, 5, 40])
@pytest.mark.parametrize("window", [None, 300])
def test_attention_plain_with_shared_keys(dtype, splits, window):
    """The plain kernel with the keys of a query divided among several blocks (more blocks than
    keys for the short sequence): the same results as with one block to a query."""
    nh, nkv, hd = 6, 2, 48
    lens, new = [1300, 3, 700], [1, 1, 2]
    qkv, kp, vp, table, seq, pos = paged_case(dtype, nh, nkv, hd, lens, new, seed=29)
    one = ops.attention_plain(qkv, nh, nkv, hd, kp, vp, table, seq, pos, 0.15, window, splits=1)
    many = ops.attention_plain(qkv, nh, nkv, hd, kp, vp, table, seq, pos, 0.15, window, splits=splits)
    close(many, one, dtype)
    auto = ops.attention_plain(qkv, nh, nkv, hd, kp, vp, table, seq, pos, 0.15, window, max_ctx_len=1300)
    close(auto, one, dtype)
    want = ref.attention_plain(qkv.cpu(), nh, nkv, hd, kp.cpu(), vp.cpu(), table.cpu(), seq.cpu(), pos.cpu(), 0.15, window)
    close(many.cpu(), want, dtype)


def test_attention_finds_one_far_key():
    """One key among hundreds is made to dominate a query's scores; the output must be that
    key's value, wherever the key lies (first page, a page edge, far back)."""
    nh, nkv, hd = 4, 2, 32
    lens, new = [600], [1]
    for far in (0, 63, 64, 300, 599):
        qkv, kp, vp, table, seq, pos = paged_case(torch.float32, nh, nkv, hd, lens, new, seed=far)
        kp.mul_(0.01)
        page = int(table[0, far // 64])
        q = qkv[0, :hd]
        kp[page, 0, far % 64, :] = q * 50.0 / (q.norm() ** 2) * math.sqrt(hd)
        got = ops.attention(qkv, nh, nkv, hd, kp, vp, table, torch.tensor([0, 1], dtype=torch.int32, device=DEV),
                            torch.tensor(lens, dtype=torch.int32, device=DEV), seq, pos, 1 / math.sqrt(hd), None, 1, 600)
        assert torch.allclose(got[0, :hd], vp[page, 0, far % 64, :], atol=1e-3), far


def test_sample_greedy_ties_and_banned():
    # wpc-runtime/src/sampling.rs:57-74
    logits = torch.tensor([[0.1, 5.0, -2.0, 4.9], [2.0, 2.0, 1.0, 2.0]], device=DEV)
    state = torch.zeros((4, 4), dtype=torch.int64, device=DEV)
    slots = torch.tensor([1, 3], dtype=torch.int32, device=DEV)
    assert ops.sample(logits, slots, state, 0.0, None).tolist() == [1, 0]
    ban = torch.tensor([1], dtype=torch.int32, device=DEV)
    assert ops.sample(logits, slots, state, 0.0, ban).tolist() == [3, 0]
    ban = torch.tensor([1, 3], dtype=torch.int32, device=DEV)
    assert ops.sample(logits, slots, state, 0.0, ban).tolist() == [0, 0]
    assert state[:, 3].tolist() == [0, 3, 0, 3]


@pytest.mark.parametrize("V", [300, 1000, 152064])
def test_sample_temperature_picks_the_cdf_index(V):
    from plain import qwen2_plain as P
    logits = rnd((3, V), seed=V, scale=2.0)
    state = torch.tensor([[0, 7, r, 5] for r in range(3)], dtype=torch.int64, device=DEV)
    slots = torch.arange(3, dtype=torch.int32, device=DEV)
    got = ops.sample(logits, slots, state, 0.8, None).tolist()
    for r in range(3):
        u = P.uniform_for(7, r, 5)
        idx, cdf, target = P.sample_temperature(logits[r].cpu().numpy(), 0.8, u)
        lo = cdf[got[r] - 1] if got[r] > 0 else 0.0
        slack = 1e-5 * cdf[-1]
        assert lo - slack <= target <= cdf[got[r]] + slack, (got[r], idx)
    assert state[:, 3].tolist() == [6, 6, 6]


def test_fill_normal_moments():
    t = torch.empty(1 << 20, dtype=torch.float32, device=DEV)
    ops.fill_normal(t, 1234, 1.0, 0.02)
    assert abs(t.mean().item() - 1.0) < 2e-4 and abs(t.std().item() - 0.02) < 2e-4
    t2 = torch.empty_like(t)
    ops.fill_normal(t2, 1235, 1.0, 0.02)
    assert not torch.equal(t, t2)


# ---- the tensor-core product against its plain twin and the torch reference ----------------------
TC_SHAPES = [(1, 128, 64), (8, 256, 128), (8, 4608, 3584), (8, 3584, 18944), (64, 1000, 520), (100, 384, 96),
             (129, 200, 72), (256, 256, 256), (300, 1000, 520), (2048, 512, 256), (513, 4608, 3584), (16, 37888, 3584),
             (2048, 3584, 1024), (1000, 5000, 520), (2100, 4608, 512),     # more tiles than SMs: persistent
             (2048, 4608, 256), (2000, 4608, 264), (2048, 3584, 264), (1024, 5000, 96)]   # 256 x 256 tiles, one wave


@pytest.mark.parametrize("shape", TC_SHAPES)
@pytest.mark.parametrize("mode", ["plain", "bias_f32out", "residual"])
@pytest.mark.parametrize("pair", [True, False])
def test_tensor_core_linear(shape, mode, pair, monkeypatch):
    """`pair` False keeps the tiles on single SMs (the kernels that sizes without pair tiles use)."""
    M, N, K = shape
    if not pair and M <= 128:
        pytest.skip("few tokens never run in pair tiles")
    monkeypatch.setattr(ops, "PAIR_TILES", pair)
    x, w = rnd((M, K), torch.bfloat16, 21), rnd((N, K), torch.bfloat16, 22, 0.05)
    swap, bn, splits = ops.plan_tensor_core_linear(M, N, K)
    if shape in ((2048, 4608, 256), (2000, 4608, 264), (2048, 3584, 264)):
        assert ops.tall_tiles(M, N, swap, bn, splits) == 256
    if mode == "plain":
        got, want = ops.linear(x, w), ops.linear_plain(x, w)
        tol = 1.2e-2
    elif mode == "bias_f32out":
        bias = rnd((N,), seed=23)
        got = ops.linear(x, w, bias, out_dtype=torch.float32)
        want = ops.linear_plain(x, w, bias, out_dtype=torch.float32)
        tol = 2e-3
    else:
        r0 = rnd((M, N), seed=24)
        got, want = ops.linear(x, w, residual=r0.clone()), ops.linear_plain(x, w, residual=r0.clone())
        tol = 2e-3
    assert ops.device_status() == 0
    err = (got.float() - want.float()).abs().max().item()
    mag = want.float().abs().max().item()
    assert err <= tol * mag, f"{shape} swap={swap} bn={bn} splits={splits}: error {err} against {mag}"
    if M <= 300 and N <= 1000:
        ref_out = ref.linear(x.cpu(), w.cpu(), None if mode == "plain" else (bias.cpu() if mode == "bias_f32out" else None),
                             out_dtype=got.dtype) if mode != "residual" else None
        if ref_out is not None:
            assert (got.cpu().float() - ref_out.float()).abs().max().item() <= tol * mag


def test_tensor_core_linear_finds_one_element():
    """Every (row, k) position reaches the right output: a single one in x picks one column of w."""
    M, N, K = 40, 300, 200
    w = rnd((N, K), torch.bfloat16, 31)
    for (m, k) in [(0, 0), (39, 199), (17, 63), (17, 64), (5, 127), (5, 128)]:
        x = torch.zeros((M, K), dtype=torch.bfloat16, device=DEV)
        x[m, k] = 1.0
        got = ops.linear(x, w, out_dtype=torch.float32)
        want = torch.zeros((M, N), device=DEV)
        want[m] = w[:, k].float()
        assert torch.equal(got, want), (m, k)


def test_tensor_core_linear_repeated_calls_share_scratch():
    x, w = rnd((8, 3584), torch.bfloat16, 41), rnd((4608, 3584), torch.bfloat16, 42, 0.05)
    first = ops.linear(x, w)
    for _ in range(3):
        assert torch.equal(ops.linear(x, w), first)


# ---- decode attention (split over CTAs) -----------------------------------------------------------
@pytest.mark.parametrize("nh,nkv,hd", [(4, 2, 16), (3, 1, 32), (4, 2, 48), (14, 2, 64), (28, 4, 128), (16, 1, 128), (2, 2, 80)])
@pytest.mark.parametrize("window", [None, 100])
@pytest.mark.parametrize("splits", [None, 1, 3, 16])
def test_attention_decode_splits(nh, nkv, hd, window, splits):
    lens, new = [1, 64, 65, 700, 333, 128], [1] * 6
    qkv, kp, vp, table, seq, pos = paged_case(torch.bfloat16, nh, nkv, hd, lens, new, seed=9)
    cu = torch.arange(7, dtype=torch.int32, device=DEV)
    ctx = torch.tensor(lens, dtype=torch.int32, device=DEV)
    scale = 1.0 / math.sqrt(hd)
    got = ops.attention(qkv, nh, nkv, hd, kp, vp, table, cu, ctx, seq, pos, scale, window, 1, max(lens), splits=splits)
    want = ref.attention_plain(qkv.cpu(), nh, nkv, hd, kp.cpu(), vp.cpu(), table.cpu(), seq.cpu(), pos.cpu(),
                               scale, window)
    close(got.cpu(), want, torch.bfloat16)


@pytest.mark.parametrize("nh,nkv,hd", [(4, 2, 16), (3, 1, 32), (4, 2, 48), (14, 2, 64), (28, 4, 128), (8, 1, 128), (2, 2, 80)])
@pytest.mark.parametrize("window", [None, 100])
@pytest.mark.parametrize("cluster,groups", [(2, 1), (3, 1), (8, 1), (16, 1), (4, 3), (2, 5), (8, 2)])
def test_attention_decode_clusters(nh, nkv, hd, window, cluster, groups):
    """Clusters of CTAs to each (sequence, kv head) pair, one or several (groups): ranks and whole
    groups without pages (a sequence of one page among eight ranks), shares that do not divide,
    every length at once."""
    lens, new = [1, 64, 65, 700, 333, 128, 1000], [1] * 7
    qkv, kp, vp, table, seq, pos = paged_case(torch.bfloat16, nh, nkv, hd, lens, new, seed=19)
    cu = torch.arange(8, dtype=torch.int32, device=DEV)
    ctx = torch.tensor(lens, dtype=torch.int32, device=DEV)
    scale = 1.0 / math.sqrt(hd)
    how = dict(cluster=cluster, groups=groups)
    got = ops.attention(qkv, nh, nkv, hd, kp, vp, table, cu, ctx, seq, pos, scale, window, 1, max(lens), **how)
    again = ops.attention(qkv, nh, nkv, hd, kp, vp, table, cu, ctx, seq, pos, scale, window, 1, max(lens), **how)
    want = ref.attention_plain(qkv.cpu(), nh, nkv, hd, kp.cpu(), vp.cpu(), table.cpu(), seq.cpu(), pos.cpu(),
                               scale, window)
    close(got.cpu(), want, torch.bfloat16)
    assert torch.equal(got, again)              # ranks and groups are added in order: the same bits every run


@pytest.mark.parametrize("cluster,groups", [(8, 1), (8, 4), (5, 3)])
def test_attention_decode_cluster_finds_one_far_key(cluster, groups):
    """One key among thousands is made to stand out; whichever rank of whichever group holds its
    page, the output is that key's value."""
    nh, nkv, hd = 28, 4, 128
    lens = [4000, 3000]
    qkv, kp, vp, table, seq, pos = paged_case(torch.bfloat16, nh, nkv, hd, lens, [1, 1], seed=23)
    cu = torch.arange(3, dtype=torch.int32, device=DEV)
    ctx = torch.tensor(lens, dtype=torch.int32, device=DEV)
    for far in (0, 63, 64, 1999, 2999):
        kp2 = kp.clone()
        for b in range(2):
            page = int(table[b, far // 64])
            kp2[page, :, far % 64, :] = 0
            kp2[page, :, far % 64, 0] = 40.0
        q2 = qkv.clone()
        q2[:, : nh * hd] = 0
        q2[:, 0 : nh * hd : hd] = 40.0                      # every head asks for element 0
        got = ops.attention(q2, nh, nkv, hd, kp2, vp, table, cu, ctx, seq, pos, 1.0, None, 1, max(lens),
                            cluster=cluster, groups=groups)
        for b in range(2):
            page = int(table[b, far // 64])
            want = vp[page, :, far % 64, :].float()            # [nkv, hd]
            out = got[b].float().view(nkv, nh // nkv, hd)
            assert (out - want[:, None, :]).abs().max().item() <= 2e-2 * want.abs().max().item() + 1e-3, (far, b)


def window_case(nh, nkv, hd, L, n_new, W, seed):
    """One sequence of L positions, the last n_new of them this step's, window W, in which two
    keys stand out for the step's last query (position L - 1, which sees L - W .. L - 1): the key
    at L - W - 1, the last one outside the window, which would win by far if it were seen, and the
    key at L - W, the first one inside, which wins among those that are.  Pages that lie wholly before the window
    of the step's first query are marked as given back (-1), as the cache leaves them."""
    qkv, kp, vp, table, seq, pos = paged_case(torch.bfloat16, nh, nkv, hd, [L], [n_new], seed=seed)
    kp.mul_(0.05)
    q2 = qkv.clone()
    q2[-1, : nh * hd] = 0
    q2[-1, 0: nh * hd: hd] = 8.0                              # every head of the last query asks for element 0
    outside, inside = L - W - 1, L - W
    for p_, height in ((outside, 60.0), (inside, 30.0)):
        page = int(table[0, p_ // 64])
        kp[page, :, p_ % 64, :] = 0
        kp[page, :, p_ % 64, 0] = height
    first_seen = max(0, (L - n_new) - W + 1)
    for block in range(first_seen // 64):
        table[0, block] = -1
    page_in = int(table[0, inside // 64])
    return q2, kp, vp, table, seq, pos, vp[page_in, :, inside % 64, :].float()


def check_window_edge(got_row, want_v, nh, nkv, hd, what):
    out = got_row.float().view(nkv, nh // nkv, hd)
    assert (out - want_v[:, None, :]).abs().max().item() <= 3e-2 * want_v.abs().max().item() + 2e-3, what


@pytest.mark.parametrize("nh,nkv,hd", [(4, 2, 64), (14, 2, 128), (2, 1, 32)])
@pytest.mark.parametrize("L,n_new,W", [(448, 150, 128), (449, 150, 128), (500, 2, 100), (700, 300, 193), (330, 200, 64)])
def test_attention_prefill_window_edges(nh, nkv, hd, L, n_new, W):
    """A window's edge in the many-token kernels (tcgen05 for head sizes 64 and 128, mma.sync
    for 32): the key just outside the window of the last query is made huge and must not be
    seen, the key just inside must win; the edge falls on a page boundary (L - W a multiple
    of 64), beside one, and inside a page; chunks of two tokens straddle it; pages before the
    window are gone from the table."""
    q2, kp, vp, table, seq, pos, want_v = window_case(nh, nkv, hd, L, n_new, W, seed=L)
    cu = torch.tensor([0, n_new], dtype=torch.int32, device=DEV)
    ctx = torch.tensor([L], dtype=torch.int32, device=DEV)
    for mma_only in (False, True):
        got = ops.attention(q2, nh, nkv, hd, kp, vp, table, cu, ctx, seq, pos, 1.0, W, n_new, L, mma_only=mma_only)
        check_window_edge(got[-1], want_v, nh, nkv, hd, (mma_only, L, n_new, W))
    # and every row against the plain kernel, which reads no page that a query cannot see
    want = ops.attention_plain(q2, nh, nkv, hd, kp, vp, table, seq, pos, 1.0, W)
    close(got, want, torch.bfloat16)
    assert ops.device_status() == 0


@pytest.mark.parametrize("nh,nkv,hd", [(4, 2, 64), (28, 4, 128), (3, 1, 48)])
@pytest.mark.parametrize("L,W", [(448, 128), (449, 128), (1000, 100), (4000, 1025), (130, 64)])
@pytest.mark.parametrize("how", ["grid", "splits", "cluster"])
def test_attention_decode_window_edges(nh, nkv, hd, L, W, how):
    """The same edge for a single-token step: the fixed grid, several CTAs to a pair, and a
    cluster to a pair."""
    q2, kp, vp, table, seq, pos, want_v = window_case(nh, nkv, hd, L, 1, W, seed=L + 1)
    cu = torch.tensor([0, 1], dtype=torch.int32, device=DEV)
    ctx = torch.tensor([L], dtype=torch.int32, device=DEV)
    kw = {"grid": dict(cluster=0), "splits": dict(splits=3), "cluster": dict(cluster=2 if W < 128 else 3)}[how]
    got = ops.attention(q2, nh, nkv, hd, kp, vp, table, cu, ctx, seq, pos, 1.0, W, 1, L, **kw)
    check_window_edge(got[0], want_v, nh, nkv, hd, (how, L, W))


@pytest.mark.parametrize("T,inner,K", [(1, 64, 96), (8, 256, 96), (50, 192, 72), (100, 320, 520), (100, 384, 520), (128, 1152, 256), (16, 4864, 896), (5, 1024, 1032), (64, 640, 2056), (200, 256, 96),
                                       (300, 384, 520), (2048, 1024, 256), (8, 18944, 3584), (2048, 2304, 256), (4096, 1152, 128)])
def test_gated_linear_fused_epilogue(T, inner, K):
    """silu(gate) * up applied by the product's epilogue (both arrangements) against the
    product followed by the activation kernel, and against torch."""
    x = rnd((T, K), torch.bfloat16, 51)
    w = rnd((2 * inner, K), torch.bfloat16, 52, 0.1 if K < 1000 else 0.02)
    got = ops.gated_linear(x, w, inner, 64)
    two = ops.silu_mul(ops.linear_plain(x, w, out_dtype=torch.float32).to(torch.bfloat16), inner, 64)
    want = ref.gated_linear(x.cpu(), w.cpu(), inner, 64)
    mag = want.float().abs().max().item()
    assert (got.cpu().float() - want.float()).abs().max().item() <= 1.5e-2 * mag
    assert (two.cpu().float() - want.float()).abs().max().item() <= 2e-2 * mag
    assert ops.device_status() == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("inner,group", [(77, 77), (256, 64), (48, 8), (40, 4)])
def test_silu_mul_groups(dtype, inner, group):
    gu = rnd((5, 2 * inner), dtype, 53, 2.0)
    close(ops.silu_mul(gu, inner, group), ref.silu_mul(gu.cpu(), inner, group).to(DEV), dtype)


@pytest.mark.parametrize("M", [65, 96, 128])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_wide_written_product_of_up_to_128_tokens(M, out_dtype):
    """65 to 128 tokens and a very wide output that is written (the output head's case): tiles on
    pairs of SMs; rows of the 256-row tile beyond the tokens are neither read nor written."""
    N, K = 256 * (ops.sms() // 2) + 72, 264
    assert ops.wide_written(M, N, False) and not ops.wide_written(M, N - 400, False) and not ops.wide_written(M, N, True)
    x, w = rnd((M, K), torch.bfloat16, 81), rnd((N, K), torch.bfloat16, 82, 0.05)
    bias = rnd((N,), seed=83)
    got = ops.linear(x, w, bias, out_dtype=out_dtype)
    want = ref.linear(x.cpu(), w.cpu(), bias.cpu(), out_dtype=torch.float32)
    mag = want.abs().max().item()
    assert (got.cpu().float() - want).abs().max().item() <= (1e-2 if out_dtype == torch.bfloat16 else 2e-3) * mag
    assert torch.equal(got, ops.linear(x, w, bias, out_dtype=out_dtype))
    assert ops.device_status() == 0


# ---- prefill attention on tcgen05 against the plain reference and the mma.sync twin ---------------
@pytest.mark.parametrize("nh,nkv,hd", [(28, 4, 128), (14, 2, 64), (4, 4, 128), (3, 1, 64), (16, 1, 128)])
@pytest.mark.parametrize("window", [None, 100])
@pytest.mark.parametrize("tiles", [1, 2])
def test_attention_prefill_tcgen05(nh, nkv, hd, window, tiles, monkeypatch):
    monkeypatch.setattr(ops, "PREFILL_ATTENTION_TILES", tiles)
    lens, new = [300, 5, 131, 700, 64], [300, 5, 31, 190, 1]
    qkv, kp, vp, table, seq, pos = paged_case(torch.bfloat16, nh, nkv, hd, lens, new, seed=11)
    cu = torch.tensor(np.concatenate([[0], np.cumsum(new)]), dtype=torch.int32, device=DEV)
    ctx = torch.tensor(lens, dtype=torch.int32, device=DEV)
    scale = 1.0 / math.sqrt(hd)
    got = ops.attention(qkv, nh, nkv, hd, kp, vp, table, cu, ctx, seq, pos, scale, window, max(new), max(lens))
    twin = ops.attention(qkv, nh, nkv, hd, kp, vp, table, cu, ctx, seq, pos, scale, window, max(new), max(lens),
                         mma_only=True)
    assert ops.device_status() == 0
    want = ref.attention_plain(qkv.cpu(), nh, nkv, hd, kp.cpu(), vp.cpu(), table.cpu(), seq.cpu(), pos.cpu(),
                               scale, window)
    close(twin.cpu(), want, torch.bfloat16)
    close(got.cpu(), want, torch.bfloat16)


def test_attention_prefill_tcgen05_growing_maximum():
    """Scores that keep growing along the sequence force the lazy rescaling of the output rows."""
    nh, nkv, hd = 2, 1, 128
    lens, new = [520], [520]
    qkv, kp, vp, table, seq, pos = paged_case(torch.bfloat16, nh, nkv, hd, lens, new, seed=12)
    for p in range(520):                      # key p points along a fixed direction, ever longer
        page = int(table[0, p // 64])
        kp[page, 0, p % 64, :] = 0.0
        kp[page, 0, p % 64, 0] = 0.25 * p
    qkv[:, 0] = 2.0
    qkv[:, hd] = 2.0
    cu = torch.tensor([0, 520], dtype=torch.int32, device=DEV)
    ctx = torch.tensor(lens, dtype=torch.int32, device=DEV)
    got = ops.attention(qkv, nh, nkv, hd, kp, vp, table, cu, ctx, seq, pos, 1.0, None, 520, 520)
    want = ref.attention_plain(qkv.cpu(), nh, nkv, hd, kp.cpu(), vp.cpu(), table.cpu(), seq.cpu(), pos.cpu(), 1.0, None)
    close(got.cpu(), want, torch.bfloat16)


# ---- few tokens, K split over the CTAs of a cluster that add up through shared memory -----------
@pytest.mark.parametrize("M", [1, 7, 16, 33, 64, 100, 128])
@pytest.mark.parametrize("N,K", [(128, 512), (200, 1032), (1000, 520), (3584, 3584), (130, 4104)])
@pytest.mark.parametrize("red_tokens", [0, 32])
def test_few_token_linear_in_clusters(M, N, K, red_tokens, monkeypatch):
    """Every split count that the plan may pick (2..8) and the three kinds of output, against the
    plain float32 product; sizes that are no multiples of the tile (weights.rs:59-78).  The
    product that adds into its output also by the older route (red.add from single CTAs)."""
    monkeypatch.setattr(ops, "RED_MAX_TOKENS", red_tokens)
    swap, bn, splits = ops.plan_tensor_core_linear(M, N, K)
    assert swap
    x, w = rnd((M, K), torch.bfloat16, 71), rnd((N, K), torch.bfloat16, 72, 0.05)
    bias = rnd((N,), seed=73)
    want = ref.linear(x.cpu(), w.cpu(), bias.cpu(), out_dtype=torch.float32)
    mag = want.abs().max().item()
    got = ops.linear(x, w, bias, out_dtype=torch.float32)
    assert (got.cpu() - want).abs().max().item() <= 2e-3 * mag, (bn, splits)
    got16 = ops.linear(x, w, bias)
    assert (got16.cpu().float() - want).abs().max().item() <= 1.2e-2 * mag
    r0 = rnd((M, N), seed=74)
    acc = ops.linear(x, w, residual=r0.clone())
    want_acc = r0.cpu() + ref.linear(x.cpu(), w.cpu(), None, out_dtype=torch.float32)
    assert (acc.cpu() - want_acc).abs().max().item() <= 2e-3 * max(mag, want_acc.abs().max().item())
    assert torch.equal(ops.linear(x, w, bias, out_dtype=torch.float32), got), "two runs differ"
    assert ops.device_status() == 0


def test_few_token_linear_in_clusters_every_slice_counts():
    """A single one in x at a k of each slice of K picks one column of w exactly: no slice is
    lost or added twice, whichever CTA of the cluster holds it."""
    M, N, K = 5, 300, 2048
    swap, bn, splits = ops.plan_tensor_core_linear(M, N, K)
    assert swap and splits >= 2, "this size is meant to be split"
    w = rnd((N, K), torch.bfloat16, 75)
    per = -(-(K // 64) // splits) * 64
    for s in range(splits):
        for k in (s * per, min(K, (s + 1) * per) - 1):
            x = torch.zeros((M, K), dtype=torch.bfloat16, device=DEV)
            x[s % M, k] = 1.0
            want = torch.zeros((M, N), device=DEV)
            want[s % M] = w[:, k].float()
            assert torch.equal(ops.linear(x, w, out_dtype=torch.float32), want), (s, k)


# ---- many tokens: 256-row tiles on pairs of SMs (tcgen05 cta_group::2) ----------------------------
@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (512, 300, 200), (400, 1000, 520), (2048, 4608, 512), (1500, 3584, 264),
                                   (3000, 520, 96)])
@pytest.mark.parametrize("width", [256, 224, 208, 144, 128])
def test_pair_tiles(M, N, K, width, monkeypatch):
    """Every tile width that the kernel takes, sizes that leave partial tiles in both
    directions, and the three kinds of output, against the float32 product (weights.rs:59-78)."""
    monkeypatch.setattr(ops, "PAIR_TILES", True)
    monkeypatch.setattr(ops, "PAIR_WIDTHS", (width,))
    assert ops.pair_tiles(M, N, False, 256)
    x, w = rnd((M, K), torch.bfloat16, 81), rnd((N, K), torch.bfloat16, 82, 0.05)
    bias = rnd((N,), seed=83)
    want = ops.linear_plain(x, w, bias, out_dtype=torch.float32)
    mag = want.abs().max().item()
    got = ops.linear(x, w, bias, out_dtype=torch.float32)
    assert (got - want).abs().max().item() <= 2e-3 * mag
    assert (ops.linear(x, w, bias).float() - want).abs().max().item() <= 1.2e-2 * mag
    r0 = rnd((M, N), seed=84)
    acc, want_acc = ops.linear(x, w, residual=r0.clone()), ops.linear_plain(x, w, residual=r0.clone())
    assert (acc - want_acc).abs().max().item() <= 2e-3 * max(mag, want_acc.abs().max().item())
    assert ops.device_status() == 0


@pytest.mark.parametrize("M,N,K", [(256, 3584, 3584), (512, 3584, 18944), (400, 1000, 2056), (2048, 896, 4864), (256, 300, 520)])
def test_pair_tiles_with_slices_of_k(M, N, K, monkeypatch):
    """Few tiles whose result is added into float32: slices of K on pairs of SMs add their shares
    with vector reductions; with and without bias, sizes that leave partial tiles and a last
    slice that is shorter."""
    assert ops.pair_tiles(M, N, False, 256)
    splits = ops.pair_splits(M, N, K)
    x, w = rnd((M, K), torch.bfloat16, 101), rnd((N, K), torch.bfloat16, 102, 0.05)
    bias = rnd((N,), seed=103)
    r0 = rnd((M, N), seed=104)
    want = ops.linear_plain(x, w, bias, residual=r0.clone())
    mag = max(want.abs().max().item(), 1.0)
    got = ops.linear(x, w, bias, residual=r0.clone())
    assert (got - want).abs().max().item() <= 2e-3 * mag, splits
    monkeypatch.setattr(ops, "PAIR_SPLIT_K", False)
    other = ops.linear(x, w, bias, residual=r0.clone())
    assert (other - want).abs().max().item() <= 2e-3 * mag
    assert ops.device_status() == 0


def test_pair_tiles_find_one_element(monkeypatch):
    """A single one in x picks one column of w exactly, for rows in either CTA of a pair and
    features in either half of the tile (each CTA holds half of the weight rows)."""
    monkeypatch.setattr(ops, "PAIR_TILES", True)
    M, N, K = 512, 600, 200
    w = rnd((N, K), torch.bfloat16, 85)
    for (m, k) in [(0, 0), (127, 63), (128, 64), (255, 199), (256, 1), (511, 130), (300, 65)]:
        x = torch.zeros((M, K), dtype=torch.bfloat16, device=DEV)
        x[m, k] = 1.0
        want = torch.zeros((M, N), device=DEV)
        want[m] = w[:, k].float()
        assert torch.equal(ops.linear(x, w, out_dtype=torch.float32), want), (m, k)


@pytest.mark.parametrize("T,inner,K", [(256, 128, 96), (2048, 1152, 256), (700, 320, 520)])
def test_pair_tiles_gated(T, inner, K, monkeypatch):
    monkeypatch.setattr(ops, "PAIR_TILES", True)
    x = rnd((T, K), torch.bfloat16, 86)
    w = rnd((2 * inner, K), torch.bfloat16, 87, 0.1)
    got = ops.gated_linear(x, w, inner, 64)
    want = ref.gated_linear(x.cpu(), w.cpu(), inner, 64)
    mag = want.float().abs().max().item()
    assert (got.cpu().float() - want.float()).abs().max().item() <= 1.5e-2 * mag
    assert ops.device_status() == 0


# ---- the q/k/v product that rotates and writes the cache in its tail ------------------------------
@pytest.mark.parametrize("nh,nkv,hd,K", [(28, 4, 128, 3584), (14, 2, 64, 896), (3, 1, 64, 520), (5, 5, 32, 1032),
                                         (8, 2, 16, 4104), (7, 1, 128, 2048)])
@pytest.mark.parametrize("new", [[1, 1, 1], [1] * 8, [6, 5, 1], [40, 3, 17, 30]])
def test_linear_qk_rope_kv_store_fused(nh, nkv, hd, K, new, monkeypatch):
    """One kernel (product in clusters, rotation and cache write in its tail) against the product
    followed by the rotation kernel, and against torch (rope.rs:24-40, model.rs:464-475).
    Several tokens of a sequence, pages that start in the middle, and sequences of one token."""
    lens = [n + off for n, off in zip(new, [70, 5, 130, 64, 0, 1, 63, 200])]
    T = sum(new)
    _, kp, vp, table, seq, pos = paged_case(torch.bfloat16, nh, nkv, hd, lens, new, seed=13)
    N = (nh + 2 * nkv) * hd
    x, w = rnd((T, K), torch.bfloat16, 91), rnd((N, K), torch.bfloat16, 92, 0.05)
    bias = rnd((N,), seed=93)
    inv = torch.tensor(np.power(1e4, -2.0 * np.arange(hd // 2) / hd), dtype=torch.float64, device=DEV)
    cos, sin = ops.rope_angles(pos, inv)
    swap, bn, splits = ops.plan_tensor_core_linear(T, N, K)
    assert swap and 2 <= splits <= 8, "this case is meant to run in clusters"
    k1, v1 = kp.clone(), vp.clone()
    q1 = ops.linear_qk_rope_kv_store(x, w, bias, nh, nkv, hd, cos, sin, k1, v1, table, seq, pos)
    assert ops.device_status() == 0
    monkeypatch.setattr(ops, "FUSE_ROPE_STORE", False)
    k2, v2 = kp.clone(), vp.clone()
    q2 = ops.linear_qk_rope_kv_store(x, w, bias, nh, nkv, hd, cos, sin, k2, v2, table, seq, pos)
    # torch: float32 product, rotation, cache write
    qkv3 = ref.linear(x.cpu(), w.cpu(), bias.cpu(), out_dtype=torch.float32)
    k3, v3 = kp.cpu().float(), vp.cpu().float()
    ref.qk_rope_kv_store(qkv3, nh, nkv, hd, cos.cpu(), sin.cpu(), k3, v3, table.cpu(), seq.cpu(), pos.cpu())
    mag = qkv3.abs().max().item()
    nq = nh * hd
    assert (q1[:, :nq].cpu().float() - qkv3[:, :nq]).abs().max().item() <= 1.2e-2 * mag
    assert (k1.cpu().float() - k3).abs().max().item() <= 1.2e-2 * mag
    assert (v1.cpu().float() - v3).abs().max().item() <= 1.2e-2 * mag
    assert (q1[:, :nq].float() - q2[:, :nq].float()).abs().max().item() <= 1.6e-2 * mag
    assert (k1.float() - k2.float()).abs().max().item() <= 1.6e-2 * mag
    # nothing but the new positions of the cache was touched
    untouched = torch.ones(kp.shape[0], 64, dtype=torch.bool)
    for t in range(T):
        b, p_ = int(seq[t]), int(pos[t])
        untouched[int(table[b, p_ // 64]), p_ % 64] = False
    assert torch.equal(k1.cpu()[untouched[:, None, :].expand(-1, nkv, -1)], kp.cpu()[untouched[:, None, :].expand(-1, nkv, -1)])
    assert torch.equal(v1.cpu()[untouched[:, None, :].expand(-1, nkv, -1)], vp.cpu()[untouched[:, None, :].expand(-1, nkv, -1)])


@pytest.mark.parametrize("nh,nkv,hd,K", [(28, 4, 128, 512), (14, 2, 64, 896), (3, 1, 64, 520), (7, 1, 128, 264)])
@pytest.mark.parametrize("new", [[256], [300, 212], [40, 600, 3, 125]])
def test_linear_qk_rope_kv_store_fused_many_tokens(nh, nkv, hd, K, new, monkeypatch):
    """The same with many tokens: the pair kernel's epilogue rotates and writes the cache."""
    lens = [n + off for n, off in zip(new, [70, 5, 130, 64])]
    T = sum(new)
    _, kp, vp, table, seq, pos = paged_case(torch.bfloat16, nh, nkv, hd, lens, new, seed=17)
    N = (nh + 2 * nkv) * hd
    x, w = rnd((T, K), torch.bfloat16, 94), rnd((N, K), torch.bfloat16, 95, 0.05)
    bias = rnd((N,), seed=96)
    inv = torch.tensor(np.power(1e4, -2.0 * np.arange(hd // 2) / hd), dtype=torch.float64, device=DEV)
    cos, sin = ops.rope_angles(pos, inv)
    swap, bn, splits = ops.plan_tensor_core_linear(T, N, K)
    if not (not swap and ops.pair_tiles(T, N, swap, bn)):
        pytest.skip("this size does not run in pair tiles")
    k1, v1 = kp.clone(), vp.clone()
    q1 = ops.linear_qk_rope_kv_store(x, w, bias, nh, nkv, hd, cos, sin, k1, v1, table, seq, pos)
    assert ops.device_status() == 0
    monkeypatch.setattr(ops, "FUSE_ROPE_STORE", False)
    k2, v2 = kp.clone(), vp.clone()
    q2 = ops.linear_qk_rope_kv_store(x, w, bias, nh, nkv, hd, cos, sin, k2, v2, table, seq, pos)
    mag = q2.float().abs().max().item()
    nq = nh * hd
    assert (q1[:, :nq].float() - q2[:, :nq].float()).abs().max().item() <= 1.6e-2 * mag
    assert (k1.float() - k2.float()).abs().max().item() <= 1.6e-2 * mag
    assert (v1.float() - v2.float()).abs().max().item() <= 1.6e-2 * mag
    # against torch on a sample of rows (the whole product in float32 on the CPU would be slow)
    rows = sorted(set([0, 1, T // 2, T - 1]))
    qkv3 = ref.linear(x.cpu()[rows], w.cpu(), bias.cpu(), out_dtype=torch.float32)
    k3, v3 = kp.cpu().float(), vp.cpu().float()
    ref.qk_rope_kv_store(qkv3, nh, nkv, hd, cos.cpu()[rows], sin.cpu()[rows], k3, v3, table.cpu(), seq.cpu()[rows], pos.cpu()[rows])
    assert (q1[rows, :nq].cpu().float() - qkv3[:, :nq]).abs().max().item() <= 1.2e-2 * mag
    for i, t in enumerate(rows):
        b, p_ = int(seq[t]), int(pos[t])
        page = int(table[b, p_ // 64])
        assert (k1[page, :, p_ % 64].cpu().float() - k3[page, :, p_ % 64]).abs().max().item() <= 1.2e-2 * mag
        assert (v1[page, :, p_ % 64].cpu().float() - v3[page, :, p_ % 64]).abs().max().item() <= 1.2e-2 * mag


# ---- the variations of the parts: another activation, another pairing, a norm per head --------------
@pytest.mark.parametrize("T,inner,K", [(1, 64, 96), (8, 256, 96), (100, 320, 520), (128, 1152, 256), (16, 4864, 896),
                                       (200, 256, 96), (300, 384, 520), (2048, 1024, 256), (77, 77, 40)])
@pytest.mark.parametrize("activation", ["silu", "gelu_tanh"])
def test_gated_linear_activations(T, inner, K, activation):
    """The activation is a parameter of the gated product: in the epilogue of every arrangement
    (few tokens in clusters and alone, tiles on one SM, tiles on pairs) and in the kernel that
    follows a plain product (sizes that the fused epilogue does not take)."""
    group = 64 if inner % 64 == 0 else inner
    x = rnd((T, K), torch.bfloat16, 151)
    w = rnd((2 * inner, K), torch.bfloat16, 152, 0.1)
    got = ops.gated_linear(x, w, inner, group, activation=activation)
    want = ref.gated_linear(x.cpu(), w.cpu(), inner, group, activation=activation)
    mag = want.float().abs().max().item()
    err = (got.cpu().float() - want.float()).abs().max().item()
    assert err <= 1.5e-2 * mag
    if activation == "gelu_tanh":          # the code is looked at: the other activation is much further away
        other = ref.gated_linear(x.cpu(), w.cpu(), inner, group, activation="silu")
        assert (got.cpu().float() - other.float()).abs().max().item() > 4 * max(err, 2e-3 * mag)
    for dtype in DTYPES:
        gu = rnd((9, 2 * inner), dtype, 153)
        close(ops.gate_mul(gu, inner, group, activation), ref.gate_mul(gu.cpu(), inner, group, activation).to(DEV), dtype)
    assert ops.device_status() == 0


def test_unknown_activation_is_refused():
    with pytest.raises(ops.KernelError, match="unknown activation"):
        ops.gated_linear(rnd((2, 64), torch.bfloat16), rnd((128, 64), torch.bfloat16), 64, 64, activation="relu")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,hd,pairs", [(3, 32, 16), (5, 48, 10), (2, 128, 64)])
def test_rope_inplace_interleaved_pairs(dtype, heads, hd, pairs):
    x = rnd((7, (heads + 1) * hd), dtype, 161)
    pos = torch.tensor([0, 1, 5, 64, 65, 1000, 31999], dtype=torch.int32, device=DEV)
    inv = torch.tensor(np.power(1e4, -2.0 * np.arange(pairs) / hd), dtype=torch.float64, device=DEV)
    cos, sin = ops.rope_angles(pos, inv)
    for inter in (False, True):
        got = ops.rope_inplace(x.clone(), heads, hd, cos, sin, interleaved=inter)
        want = ref.rope_inplace(x.cpu().clone(), heads, hd, cos.cpu(), sin.cpu(), interleaved=inter)
        close(got.cpu(), want, dtype)
        assert torch.equal(got[:, heads * hd:], x[:, heads * hd:])          # the head behind is left alone
    a = ops.rope_inplace(x.clone(), heads, hd, cos, sin, interleaved=False)
    b = ops.rope_inplace(x.clone(), heads, hd, cos, sin, interleaved=True)
    assert not torch.equal(a, b)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,hd", [(3, 32), (5, 48), (28, 128), (1, 20)])
def test_head_rmsnorm(dtype, heads, hd):
    x = rnd((11, (heads + 2) * hd), dtype, 171)
    gain = 1.0 + rnd((hd,), torch.float32, 172, 0.1)
    got = ops.head_rmsnorm_(x.clone(), heads, hd, gain, 1e-5)
    want = ref.head_rmsnorm_(x.cpu().clone(), heads, hd, gain.cpu(), 1e-5)
    close(got.cpu(), want, dtype)
    assert torch.equal(got[:, heads * hd:], x[:, heads * hd:])
    # a view that starts behind other heads, as the k heads of a q/k/v row do
    view = x.clone()
    ops.head_rmsnorm_(view[:, hd:], heads, hd, gain, 1e-5)
    want2 = x.cpu().clone()
    ref.head_rmsnorm_(want2[:, hd:], heads, hd, gain.cpu(), 1e-5)
    close(view.cpu(), want2, dtype)
