"""The entry point for callers that cannot allocate device memory (csrc/no_alloc.h), called
through its exported C symbol the way such a caller would: raw addresses in, no torch
allocator behind it.  Such callers are embedders whose host owns all device memory, or loops
that cannot afford an allocation's latency; for them the split-K product keeps its scratch in
a fixed array inside the library.  Its output is compared with the library's ordinary product
(`ops.linear`, whose scratch comes from torch's allocator), on two calls in a row of different
sizes, because the second call sees whatever the first left in the shared array.  Named to be
collected last."""
import ctypes

import pytest
import torch

from wpc_engine_b200 import ops

pytestmark = pytest.mark.gpu


def call_static(lib, x, w, bias, out, splits=0):
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    return lib.wpc_linear_few_tokens_static(
        ctypes.c_void_p(x.data_ptr()), x.stride(0), x.shape[0], ctypes.c_void_p(w.data_ptr()), w.stride(0),
        w.shape[0], x.shape[1], ctypes.c_void_p(0 if bias is None else bias.data_ptr()),
        ctypes.c_void_p(out.data_ptr()), 1 if out.dtype == torch.bfloat16 else 0, out.stride(0), splits, stream)


def read_status(lib):
    word = ctypes.c_int(-1)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert lib.wpc_linear_few_tokens_static_status(ctypes.byref(word), stream) == 0
    return word.value


def test_static_scratch_entry_point_matches_the_ordinary_one_twice_in_a_row():
    lib = ops.library()
    g = torch.Generator().manual_seed(7)
    cases = [(8, 4608, 3584, torch.bfloat16, True), (40, 3584, 2048, torch.float32, False)]
    # One call of each tile width first: the first call on a device looks up the array's address,
    # and the first launch of a kernel lets the driver bring its code onto the device, which
    # takes device memory that is nobody's allocation.
    for tokens in (8, 40):
        warm = torch.zeros((tokens, 64), dtype=torch.bfloat16, device="cuda")
        assert call_static(lib, warm, torch.zeros((128, 64), dtype=torch.bfloat16, device="cuda"), None,
                           torch.empty((tokens, 128), dtype=torch.bfloat16, device="cuda")) == 0
    torch.cuda.synchronize()
    for tokens, features, K, out_dtype, with_bias in cases:
        x = torch.randn((tokens, K), generator=g).to(torch.bfloat16).cuda()
        w = (torch.randn((features, K), generator=g) * 0.05).to(torch.bfloat16).cuda()
        bias = torch.randn((features,), generator=g).cuda() if with_bias else None
        out = torch.empty((tokens, features), dtype=out_dtype, device="cuda")    # the caller's own memory
        torch.cuda.synchronize()
        # free bytes as the driver counts them: an allocation by anybody in this process would
        # show, not only one by torch's allocator
        free_before, _ = torch.cuda.mem_get_info()
        held_before = torch.cuda.memory_allocated()
        rc = call_static(lib, x, w, bias, out)
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free_before
        assert torch.cuda.memory_allocated() == held_before
        assert read_status(lib) == 0
        want = ops.linear(x, w, bias, out_dtype=out_dtype)
        err = (out.float() - want.float()).abs().max().item()
        tol = 1.2e-2 if out_dtype == torch.bfloat16 else 2e-3
        assert err <= tol * want.float().abs().max().item(), (tokens, features, K, err)


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    lib = ops.library()
    x = torch.zeros((128, 512), dtype=torch.bfloat16, device="cuda")
    w = torch.zeros((128 * 40, 512), dtype=torch.bfloat16, device="cuda")
    out = torch.empty((128, w.shape[0]), dtype=torch.bfloat16, device="cuda")
    assert call_static(lib, x, w, None, out, splits=8) == 1003       # 40 tiles * 8 * 128 * 128 floats > 1 Mi
    assert call_static(lib, x, w, None, out, splits=0) == 0          # the call's own choice fits
    big = torch.zeros((128 * 1025, 64), dtype=torch.bfloat16, device="cuda")
    out2 = torch.empty((1, big.shape[0]), dtype=torch.bfloat16, device="cuda")
    assert call_static(lib, x[:1, :64].contiguous(), big, None, out2) == 1003   # more tiles than tickets
    assert call_static(lib, x, w, None, out, splits=-1) == 1001                  # no such split
    torch.cuda.synchronize()


def test_static_scratch_entry_point_reports_a_kernel_that_gave_up():
    """The entry point's own status word: a caller reads it through the library, and the next
    call does not wipe it.  The wait is made to run out the harmless way (see test_status_gpu.py)."""
    lib = ops.library()
    x = torch.ones((4, 1024), dtype=torch.bfloat16, device="cuda")
    w = torch.ones((256, 1024), dtype=torch.bfloat16, device="cuda")
    out = torch.zeros((4, 256), dtype=torch.float32, device="cuda")
    assert read_status(lib) == 0
    ops.set_wait_policy(3_000_000, starve=True)
    try:
        assert call_static(lib, x, w, None, out) == 0
        torch.cuda.synchronize()
    finally:
        ops.set_wait_policy()
    assert call_static(lib, x, w, None, out) == 0          # an ordinary call behind it: the word stays
    assert read_status(lib) == 1004
    assert read_status(lib) == 0                           # reading cleared it
    assert torch.equal(out, torch.full((4, 256), 1024.0, device="cuda"))
