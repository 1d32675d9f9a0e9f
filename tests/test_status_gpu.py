"""A kernel that gave up is an error, not a result.

Every wait of a kernel on one of its barriers is bounded; when it runs out the kernel records
1004 in the device status word, frees what it holds and returns.  These tests make that
happen the one way that harms nothing: the library's `starve` switch keeps the warp that
starts a kernel's TMA copies from starting any, so the barriers that wait for data are never
signalled (nothing is in flight, nothing traps or spins without bound), and the wait limit is
set to a few milliseconds.  They check that the call returns, that the word says 1004, that the
step function and the generation loop raise, that a failed step leaves the cache as it was,
and that the next ordinary call on the same stream is right (tensor memory was freed,
tickets are clean)."""
import numpy as np
import pytest
import torch

from conftest import make_folder
from helpers import assert_close_to_plain, random_tokens, run_whole
from wpc_engine_b200 import Engine, GenerationOptions, KernelError, SequenceStep, generate, ops

import torch_ops as ref

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture
def starved():
    """Kernels with TMA producers start no copies and give up after 3 ms."""
    ops.clear_device_status()
    ops.set_wait_policy(3_000_000, starve=True)
    try:
        yield
    finally:
        ops.set_wait_policy()
        torch.cuda.synchronize()
        ops.clear_device_status()


def product_inputs(tokens, features, K, seed=0):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn((tokens, K), generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn((features, K), generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    return x, w


def check_product(x, w, residual=False):
    if residual:
        base = torch.randn((x.shape[0], w.shape[0]), device=DEV)
        got = ops.linear(x, w, residual=base.clone())
        want = ref.linear(x, w, residual=base.clone())
    else:
        got, want = ops.linear(x, w, out_dtype=torch.float32), ref.linear(x, w, out_dtype=torch.float32)
    assert (got - want).abs().max().item() <= 2e-2 * want.abs().max().item()


# (tokens, features, K, added into a float32 residual, clusters allowed): few tokens with the
# slices of K in a cluster; the same through scratch memory and tickets; slices that add their
# shares with red.add; a tile to a CTA; split tiles of the normal arrangement with tickets; one
# persistent CTA to an SM; 256 x 256 tiles on pairs of SMs
PRODUCTS = [(8, 1024, 2048, False, True), (8, 1024, 2048, False, False), (8, 256, 2048, True, True),
            (300, 512, 256, False, True), (200, 4864, 512, False, True), (300, 12800, 128, False, True),
            (512, 1024, 512, False, True)]


@pytest.mark.parametrize("tokens,features,K,residual,clusters", PRODUCTS)
def test_a_starved_product_returns_with_1004_and_the_next_one_is_right(starved, monkeypatch, tokens, features, K,
                                                                       residual, clusters):
    monkeypatch.setattr(ops, "CLUSTER_SPLITS", clusters)
    x, w = product_inputs(tokens, features, K)
    check = lambda: check_product(x, w, residual)
    ops.set_wait_policy()               # first the ordinary product, so that a wrong size shows here
    check()
    assert ops.device_status() == 0
    ops.set_wait_policy(3_000_000, starve=True)
    if residual:
        ops.linear(x, w, residual=torch.zeros((tokens, features), device=DEV))
    else:
        ops.linear(x, w, out_dtype=torch.float32)
    torch.cuda.synchronize()            # the call comes back
    assert ops.device_status() == 1004
    with pytest.raises(KernelError, match="1004"):
        ops.check_device_status()
    assert ops.device_status() == 0     # raising cleared it
    ops.set_wait_policy()
    for _ in range(2):                  # tensor memory was freed and the tickets are clean
        check()
    assert ops.device_status() == 0


def test_a_starved_gated_product_and_qkv_tail(starved):
    ops.set_wait_policy()
    x, w = product_inputs(8, 2 * 1024, 1024, seed=3)
    want = ops.gated_linear(x, w, 1024, 64)
    ops.set_wait_policy(3_000_000, starve=True)
    ops.gated_linear(x, w, 1024, 64)
    torch.cuda.synchronize()
    assert ops.device_status() == 1004
    ops.clear_device_status()
    ops.set_wait_policy()
    assert torch.equal(ops.gated_linear(x, w, 1024, 64), want)
    assert ops.device_status() == 0


def attention_case(hd=64, n_new=300, nh=4, nkv=2):
    g = torch.Generator().manual_seed(11)
    n_pages = (n_new + 63) // 64
    q = torch.randn((n_new, nh * hd), generator=g).to(torch.bfloat16).to(DEV)
    k_pages = torch.randn((n_pages, nkv, 64, hd), generator=g).to(torch.bfloat16).to(DEV)
    v_pages = torch.randn((n_pages, nkv, 64, hd), generator=g).to(torch.bfloat16).to(DEV)
    table = torch.arange(n_pages, dtype=torch.int32, device=DEV).view(1, -1)
    cu = torch.tensor([0, n_new], dtype=torch.int32, device=DEV)
    ctx = torch.tensor([n_new], dtype=torch.int32, device=DEV)
    seq = torch.zeros(n_new, dtype=torch.int32, device=DEV)
    pos = torch.arange(n_new, dtype=torch.int32, device=DEV)
    args = (q, nh, nkv, hd, k_pages, v_pages, table, cu, ctx, seq, pos, hd ** -0.5, None, n_new, n_new)
    return args


@pytest.mark.parametrize("hd", [64, 128])
def test_a_starved_prefill_attention_returns_with_1004_and_the_next_one_is_right(starved, hd):
    args = attention_case(hd)
    ops.set_wait_policy()
    want = ref.attention(*args).float()
    ok = lambda: (ops.attention(*args).float() - want).abs().max().item() <= 3e-2 * want.abs().max().item()
    assert ok()
    ops.set_wait_policy(3_000_000, starve=True)
    ops.attention(*args)
    torch.cuda.synchronize()
    assert ops.device_status() == 1004
    ops.clear_device_status()
    ops.set_wait_policy()
    assert ok() and ok()
    assert ops.device_status() == 0


MEDIUM = dict(architectures=["Qwen2ForCausalLM"], num_hidden_layers=2, hidden_size=512, num_attention_heads=8,
              num_key_value_heads=2, head_dim=64, intermediate_size=1024, vocab_size=700, rope_theta=1e6,
              rms_norm_eps=1e-6, max_position_embeddings=2048, tie_word_embeddings=False)


def test_step_and_generate_raise_and_leave_the_cache_as_it_was(starved, tmp_path_factory):
    ops.set_wait_policy()
    folder = make_folder(tmp_path_factory, MEDIUM, 81, torch.bfloat16)
    eng = Engine.from_folder(folder, dtype="bfloat16", max_tokens=2048)
    req = random_tokens(700, 300, 1400)
    slot = eng.open_sequence()
    eng.step([SequenceStep(slot, req[:100], want=[])])
    held = eng.cache.groups[0].pool.n_held
    ops.set_wait_policy(3_000_000, starve=True)
    with pytest.raises(KernelError, match="wait inside a kernel ran out"):
        eng.step([SequenceStep(slot, req[100:300], want=[199])])
    assert eng.sequence_length(slot) == 100 and eng.cache.groups[0].pool.n_held == held
    eng.cache.check()
    with pytest.raises(KernelError):
        generate(eng, [req[:40], req[40:70]], GenerationOptions(max_tokens=4))
    assert eng.cache.slots.n_held == 1            # generate gave its slots back
    ops.set_wait_policy()
    # the same engine goes on where it was: the failed step left nothing behind
    out = eng.step([SequenceStep(slot, req[100:300], want=list(range(200)))]).float().cpu().numpy()
    eng.close_sequence(slot)
    want = run_whole(eng, req)
    assert np.abs(out - want[100:]).max() <= 3e-2 * np.abs(want).max()
    assert_close_to_plain(want, folder, req, "bfloat16", "after the failures")
    assert generate(eng, [req[:40]], GenerationOptions(max_tokens=4)) == generate(eng, [req[:40]], GenerationOptions(max_tokens=4))
    eng.cache.check()


def test_a_status_word_set_by_anything_stops_the_step_and_the_loop(folders):
    """The host side alone: the word is set by the test, as a kernel would have set it."""
    ops.clear_device_status()
    eng = Engine.from_folder(folders[("A", "float32")], dtype="float32", max_tokens=512)
    slot = eng.open_sequence()
    ops.status_word().fill_(1004)
    with pytest.raises(KernelError, match="1004"):
        eng.step([SequenceStep(slot, [1, 2, 3], want=[2])])
    assert eng.sequence_length(slot) == 0 and ops.device_status() == 0
    assert eng.step([SequenceStep(slot, [1, 2, 3], want=[2])]).shape == (1, 256)
    ops.status_word().fill_(1001)
    assert eng.step([SequenceStep(slot, [4], want=[0])], check=False) is not None     # the caller looks later
    with pytest.raises(KernelError, match="no page"):
        ops.check_device_status()
    eng.close_sequence(slot)
    ops.status_word().fill_(1004)
    with pytest.raises(KernelError, match="1004"):
        generate(eng, [[5, 6, 7], [8]], GenerationOptions(max_tokens=5))
    assert eng.cache.slots.n_held == 0 and ops.device_status() == 0
    assert len(generate(eng, [[5, 6, 7], [8]], GenerationOptions(max_tokens=5))[1]) == 5


def test_a_position_without_a_page_is_reported(folders):
    """The cache write of a token whose position has no page is dropped by the kernel and shows
    in the status word (the engine never builds such a table; this one is made by hand)."""
    ops.clear_device_status()
    for dtype in (torch.float32, torch.bfloat16):
        nh, nkv, hd, T = 2, 1, 32, 3
        qkv = torch.randn((T, (nh + 2 * nkv) * hd), device=DEV).to(dtype)
        pages = torch.zeros((2, nkv, 64, hd), dtype=dtype, device=DEV)
        table = torch.tensor([[0, -1]], dtype=torch.int32, device=DEV)
        seq = torch.zeros(T, dtype=torch.int32, device=DEV)
        pos = torch.tensor([5, 64, 6], dtype=torch.int32, device=DEV)       # position 64 lies in block 1: no page
        ops.qk_rope_kv_store(qkv, nh, nkv, hd, None, None, pages, pages.clone(), table, seq, pos)
        assert ops.device_status() == 1001
        ops.clear_device_status()
