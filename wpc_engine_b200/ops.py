"""The device operations that the parts call: each checks its arguments and launches one
hand-written kernel of the in-tree CUDA library on the current stream.

There is no fallback: without a CUDA device, or if the library cannot be built or loaded,
every operation raises `KernelError`.  Tensors are passed by address through the library's C
interface (csrc/api.h); outputs are allocated here with torch's allocator, which is all that
torch does on this path.
"""
from __future__ import annotations

import ctypes
import os
import threading
from typing import Optional, Tuple

import torch

from .constants import PAGE

_F32, _BF16 = 0, 1
_ERRORS = {1001: "bad argument", 1002: "unsupported size", 1003: "size beyond the stated maximum",
           1004: "a device-side wait ran out"}
# what a non-zero device status word means (written by kernels, read by the host after them)
_DEVICE_ERRORS = {1001: "a token's position has no page in the cache (its key and value were not written)",
                  1004: "a wait inside a kernel ran out; the kernel returned without finishing its output"}


class KernelError(RuntimeError):
    """A kernel could not be launched, or the kernel library is missing."""


_lib = None
_lib_lock = threading.Lock()


def library():
    """The loaded kernel library (built on first use)."""
    global _lib
    if _lib is None:
        with _lib_lock:
            if _lib is None:
                from .csrc.build import BuildError, library_path
                try:
                    path = library_path()
                    _lib = ctypes.CDLL(path)
                except (BuildError, OSError) as e:
                    raise KernelError(f"the CUDA kernel library is not available: {e}") from None
    return _lib


def set_wait_policy(limit_ns: int = 2_000_000_000, starve: bool = False) -> None:
    """How long a kernel waits on one of its barriers before it gives up and records an error
    in the device status word (2 s by default).  `starve` is for tests of that path: kernels
    with TMA producers then start no copies, so that their waits run out."""
    _check("set_wait_policy", library().wpc_set_wait_policy(ctypes.c_ulonglong(int(limit_ns)), int(bool(starve))))


def set_pdl(on: bool) -> bool:
    """Programmatic dependent launch for all kernels, on by default; returns the old setting."""
    return bool(library().wpc_set_pdl(int(bool(on))))


def set_decode_early_pages(on: bool) -> bool:
    """Whether decode attention starts copying the pages of earlier positions while the kernel
    ahead of it still runs (on by default); returns the old setting."""
    return bool(library().wpc_attention_decode_early_pages(int(bool(on))))


def require_device(device="cuda") -> None:
    """Raises unless `device` is a CUDA device and the kernel library loads."""
    dev = torch.device(device)
    if dev.type != "cuda":
        raise KernelError(f"this engine runs on CUDA devices only, not on {dev}")
    if not torch.cuda.is_available():
        raise KernelError("no CUDA device is available; there is no CPU path")
    library()


def _code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return _F32
    if dtype == torch.bfloat16:
        return _BF16
    raise KernelError(f"unsupported element type {dtype}")


def _p(t: Optional[torch.Tensor]):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


launch_count = 0          # kernels launched through this module (graph replays are counted by the engine)


def _check(name: str, rc: int) -> None:
    global launch_count
    launch_count += 1
    if rc == 0:
        return
    if rc in _ERRORS:
        raise KernelError(f"{name}: {_ERRORS[rc]}")
    raise KernelError(f"{name}: CUDA error {rc}")


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise KernelError(msg)


def _rows(t: torch.Tensor, name: str) -> None:
    _need(t.is_cuda, f"{name} must be on a CUDA device")
    _need(t.dim() == 2 and t.stride(1) == 1, f"{name} must be a matrix with unit column stride")


# ---------------------------------------------------------------------------------------------
def embed(tokens: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """float32 [T, width] = table[tokens]."""
    _need(tokens.dtype == torch.int32 and tokens.is_contiguous(), "tokens must be contiguous int32")
    _need(table.is_contiguous(), "the embedding table must be contiguous")
    T, (V, H) = tokens.numel(), table.shape
    out = torch.empty((T, H), dtype=torch.float32, device=table.device)
    _check("embed", library().wpc_embed(_p(tokens), _p(table), _code(table.dtype), _p(out), T, H, V, _stream()))
    return out


def rmsnorm(x: torch.Tensor, gain: torch.Tensor, eps: float, out_dtype: torch.dtype,
            rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x * rsqrt(mean(x^2) + eps) * gain per row; x and gain float32.  With `rows` (int32 [n]) only
    the rows x[rows[i]] are normed, into [n, width]: the gather and the norm in one kernel."""
    _need(x.dtype == torch.float32 and x.is_contiguous() and x.dim() == 2, "x must be contiguous float32 [T, width]")
    _need(gain.dtype == torch.float32 and gain.numel() == x.shape[1], "gain must be float32 [width]")
    n = x.shape[0]
    if rows is not None:
        _need(rows.dtype == torch.int32 and rows.is_contiguous(), "rows must be contiguous int32")
        n = rows.numel()
    out = torch.empty((n, x.shape[1]), dtype=out_dtype, device=x.device)
    _check("rmsnorm", library().wpc_rmsnorm(_p(x), _p(gain), ctypes.c_float(eps), _p(out), _code(out_dtype),
                                            x.shape[0], x.shape[1], _p(rows), n, _stream()))
    return out


def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
           out_dtype: Optional[torch.dtype] = None, residual: Optional[torch.Tensor] = None,
           plain: bool = False, static_weight: bool = False) -> torch.Tensor:
    """x [T, K] times w [N, K] transposed, plus bias (float32 [N]).  With `residual` (float32
    [T, N], contiguous) the result is added to it in place in float32 and it is returned.

    bfloat16 x and w go to the tensor-core kernel (csrc/gemm_tc.cu) when their layout allows
    TMA (16-byte aligned rows); everything else, and everything with `plain`, runs on the
    CUDA cores in float32 (csrc/gemm_simt.cu).  `static_weight` promises that w is a model
    parameter that no earlier work still in flight writes; the tensor-core kernel then fetches
    its first tiles while the kernel before it is still finishing."""
    _rows(x, "x")
    _rows(w, "w")
    M, K = x.shape
    N = w.shape[0]
    _need(w.shape[1] == K, f"x has {K} columns, w has {w.shape[1]}")
    if bias is not None:
        _need(bias.dtype == torch.float32 and bias.numel() == N and bias.is_contiguous(), "bias must be float32 [N]")
    if residual is not None:
        _need(residual.dtype == torch.float32 and residual.shape == (M, N) and residual.is_contiguous(),
              "residual must be contiguous float32 [T, N]")
        out, accumulate = residual, 1
    else:
        out = torch.empty((M, N), dtype=out_dtype or x.dtype, device=x.device)
        accumulate = 0
    if M == 0:
        return out
    if not plain and _tensor_core_linear(x, w, bias, out, accumulate, static_weight):
        return out
    _check("gemm_simt", library().wpc_gemm_simt(
        _p(x), _code(x.dtype), x.stride(0), _p(w), _code(w.dtype), w.stride(0), _p(bias), _p(out),
        _code(out.dtype), out.stride(0), accumulate, M, N, K, _stream()))
    return out


def linear_plain(x, w, bias=None, out_dtype=None, residual=None) -> torch.Tensor:
    """The same product on the CUDA cores only (the plain twin of `linear`)."""
    return linear(x, w, bias, out_dtype, residual, plain=True)


_SMS = 148                # SMs of a B200, which the launch plans were measured on
_sms_of = {}


def sms() -> int:
    """SMs of the current device (148 where there is none, for the plans' arithmetic alone)."""
    if not torch.cuda.is_available():
        return _SMS
    dev = torch.cuda.current_device()
    if dev not in _sms_of:
        _sms_of[dev] = int(torch.cuda.get_device_properties(dev).multi_processor_count)
    return _sms_of[dev]


# Switches between kernels for the same product.  The defaults are the measured best on B200;
# the tests flip them to reach the kernels that the defaults leave for other sizes.
PAIR_TILES = True         # many tokens: 256 x 256 tiles on pairs of SMs (tcgen05 cta_group::2)
CLUSTER_SPLITS = True     # the CTAs that split one tile's K form a cluster and add up through shared memory
# A cluster holds at most 8 slices of K.  A product that adds into the float32 residual with at
# most RED_MAX_TOKENS tokens and so few tiles that its clusters would leave more than half of the
# SMs idle takes the older scheme instead: up to 16 slices, one CTA to an SM, deep rings, the
# slices add their shares with red.global.add (the last bits of the sum then depend on the
# order of arrival).  Measured at the 0.5B shape, 16 sequences: down_proj (7 tiles) as 112 CTAs
# against 56 in clusters, a step takes 0.84 against 0.94 ms; o_proj, 21 CTAs either way, 0.94
# against 0.97 ms (the cluster's tail is the longer one).  With more tiles the cluster product
# wins, two CTAs to an SM beside the attention clusters that end together (o_proj of the 7B
# shape: a step at batch 8 3.15 against 3.18 ms, batch 1 2.87 against 2.91 ms), and the atomics
# grow with the token count (64 tokens: 25.5 against 14.8 us).
RED_MAX_TOKENS = 32
RED_MAX_K_BLOCKS = 128
_WORKSPACE_FLOATS = 8 << 20        # 32 MiB of split-K partial sums
_WORKSPACE_COUNTERS = 4096
_workspaces = {}


def workspace(device):
    """(scratch float32, ticket counters int32, status int32) of a device, allocated once.
    Kernels that use them run one after another on a stream; calls on several streams at
    once would share them and race."""
    key = torch.device(device).index or 0
    ws = _workspaces.get(key)
    if ws is None:
        ws = (torch.empty(_WORKSPACE_FLOATS, dtype=torch.float32, device=device),
              torch.zeros(_WORKSPACE_COUNTERS, dtype=torch.int32, device=device),
              torch.zeros(1, dtype=torch.int32, device=device))
        _workspaces[key] = ws
    return ws


def status_word(device="cuda") -> torch.Tensor:
    """The device error word itself (int32 [1]), for callers that copy it beside their results."""
    return workspace(device)[2]


def device_status(device="cuda") -> int:
    """The device error word (0: none), read now: it waits for the device.  Kernels set it when
    a bounded wait ran out (1004) or a position had no page (1001); it keeps the last error
    until `raise_device_status` or `clear_device_status`."""
    ws = _workspaces.get(torch.device(device).index or 0)
    return 0 if ws is None else int(ws[2].item())


def clear_device_status(device="cuda") -> None:
    ws = _workspaces.get(torch.device(device).index or 0)
    if ws is not None:
        ws[2].zero_()


def raise_device_status(code: int, device="cuda", what: str = "a kernel") -> None:
    """Turns a non-zero status word (already read) into a KernelError and clears the word."""
    if code:
        clear_device_status(device)
        raise KernelError(f"{what} reported error {code}: {_DEVICE_ERRORS.get(code, 'unknown code')}")


def check_device_status(device="cuda", what: str = "a kernel") -> None:
    """Reads the status word (waits for the device) and raises KernelError if it is set."""
    raise_device_status(device_status(device), device, what)


_cluster_capacity = {}


def cluster_capacity(bn: int, splits: int) -> int:
    """How many clusters of `splits` CTAs of the few-token kernel run side by side (asked once)."""
    key = (bn, splits)
    if key not in _cluster_capacity:
        _cluster_capacity[key] = max(0, int(library().wpc_gemm_tc_cluster_capacity(bn, splits)))
    return _cluster_capacity[key]


def plan_tensor_core_linear(M: int, N: int, K: int):
    """(swap, bn, splits) for x [M, K] . w [N, K]^T.  Few tokens: the weights take the MMA's
    128 rows and the tokens its columns (swap).  Few tiles: K is split over CTAs so that
    about all SMs stream weights.  With few tokens the CTAs of a tile form a cluster (at most
    8) that adds the slices up through shared memory: the split is the largest for which all
    clusters run at once."""
    k_blocks = (K + 63) // 64
    if M <= 128:
        swap, bn = True, (16 if M <= 16 else 32 if M <= 32 else 64 if M <= 64 else 128)
        tiles = (N + 127) // 128
    else:
        swap = False
        m_tiles = (M + 127) // 128
        bn = 256 if N >= 256 else 128 if N > 64 else 64
        tiles = m_tiles * ((N + bn - 1) // bn)
    splits = 1
    if tiles * 2 <= sms():
        if swap and CLUSTER_SPLITS:
            for s in range(min(8, k_blocks // 4), 1, -1):
                if tiles <= cluster_capacity(bn, s):
                    splits = s
                    break
            return swap, bn, splits
        splits = _ticket_splits(tiles, k_blocks, bn)
    return swap, bn, splits


def _ticket_splits(tiles: int, k_blocks: int, bn: int) -> int:
    """Slices of K for products that combine through scratch memory or red.add: about one CTA
    to an SM (two to an SM measured slower in a whole step, also with many tokens)."""
    splits = max(1, min(sms() // tiles, k_blocks // 4, 16))
    while splits > 1 and tiles * splits * bn * 128 > _WORKSPACE_FLOATS:
        splits -= 1
    if tiles > _WORKSPACE_COUNTERS:
        splits = 1
    return splits


def tall_tiles(M: int, N: int, swap: bool, bn: int, splits: int, K: int = 0, accumulate: bool = False) -> int:
    """The width of 256-row tiles for this product (256), or 0 to keep 128 x bn tiles.  In a
    256-row tile two MMAs share each weight tile (a third less operand traffic per flop).  They
    are used when all tiles make a single wave that covers at least half of the SMs.  Measured
    at 2,048 tokens of the 7B shape: qkv 1.36 against 1.19 PFLOP/s, down 1.20 against 1.05.
    With more tiles than SMs the 128 x 256 tiles win, because their epilogue overlaps the next
    tile (1.27 against 0.94 PFLOP/s at 8,192 tokens); a product that adds into the residual
    stream with a short K keeps them too (its read-modify-write epilogue is not hidden in a
    tall tile: 0.73 against 0.78); narrower tall tiles that would fill the wave better (208
    wide for 3584 features) were slower (0.47 and 1.09 against 0.78 and 1.20)."""
    if swap or bn != 256 or splits != 1 or M < 256 or (accumulate and K < 8192):
        return 0
    tiles = ((M + 255) // 256) * ((N + 255) // 256)
    return 256 if sms() // 2 <= tiles <= sms() else 0


def pair_tiles(M: int, N: int, swap: bool, bn: int, padded: bool = True) -> bool:
    """Whether the product runs in 256-row tiles on pairs of SMs (tcgen05 cta_group::2, each SM
    fetches a third less per flop than with 128 x 256 tiles of its own): more than 128 tokens
    and a wide output.  `padded` False (the gated product, by far the largest of a layer):
    only token counts that 256-row tiles do not pad much further than 128-row tiles.  Measured
    at the 7B shape, pair tiles against 128-row tiles: 300 tokens o_proj 18.7 against 28.4 us,
    down 54 against 66, q/k/v 33.0 against 35.6, but gate/up 132 against 99 us; 1,030 tokens
    q/k/v 52 against 63 us, down 126 against 136, gate/up 242 against 240."""
    if not (PAIR_TILES and not swap and bn == 256 and M > 128):
        return False
    return bool(padded or (M >= 256 and (M % 256 == 0 or M % 256 > 128)))


def wide_written(M: int, N: int, accumulate) -> bool:
    """65 to 128 tokens and an output that is written (not added to) and so wide that 256-wide
    tiles fill the pairs of SMs at least once (the output head): tiles on pairs of SMs instead
    of the few-token arrangement, in which every 128 features fetch the tokens again.  Measured
    at the 7B shape's head: 215 against 262 us at 96 tokens, 223 against 288 us at 128."""
    return bool(PAIR_TILES and 64 < M <= 128 and not accumulate and -(-N // 256) >= sms() // 2)


PAIR_WIDTHS = (256,)      # tile widths that pair_tile_width may choose from (the kernel takes 128..256 in steps of 16)


def pair_tile_width(M: int, N: int) -> int:
    """Columns of a pair's tile: the width whose tiles fill whole waves of the pairs of SMs best.
    Only 256 is offered: narrower tiles keep more pairs busy in a part-empty last wave, but a
    pair takes in its operands at about 83 GB/s per SM whatever the width, so a wave of 160-wide
    tiles costs 86 % of a wave of 256-wide ones for 62 % of the work (measured at 2,048 x 3,584:
    one width of 256: 227 us for K = 18,944; 9 tile columns of 256 and then 8 of 160 as two
    launches, both single full waves: 248 us)."""
    tiles_m = (M + 255) // 256
    best, best_cost = 256, None
    for pn in PAIR_WIDTHS:
        waves = -(-(tiles_m * -(-N // pn)) // (sms() // 2))
        cost = waves * (pn + 32)
        if best_cost is None or cost < best_cost:
            best, best_cost = pn, cost
    return best


PAIR_SPLIT_K = True


def pair_splits(M: int, N: int, K: int) -> int:
    """Slices of K for a product in 256 x 256 tiles on pairs of SMs that adds into a float32
    output: as many as keep every pair busy once, each at least 4 blocks of 64 deep, 8 at most.
    The slices add their shares with 16-byte reductions.  Measured at the 7B shape against 128 x
    256 tiles on single SMs whose slices add value by value: 256 tokens o_proj 15.4 against 25.6 us
    and down 33.8 against 50.4 us; 512 tokens 19.7 against 32.2 and 58.2 against 86.5 us."""
    tiles = -(-M // 256) * -(-N // 256)
    return max(1, min((sms() // 2) // max(tiles, 1), ((K + 63) // 64) // 4, 8))


def _tensor_core_linear(x, w, bias, out, accumulate, static_weight=False) -> bool:
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        return False
    M, K = x.shape
    N = w.shape[0]
    if K % 8 or x.stride(0) % 8 or w.stride(0) % 8 or x.data_ptr() % 16 or w.data_ptr() % 16:
        return False
    swap, bn, splits = plan_tensor_core_linear(M, N, K)
    wide = wide_written(M, N, accumulate)
    if wide:
        swap, bn, splits = False, 256, 1
    if not swap and not accumulate:
        # Many tokens and an output that is written, not added to: K stays whole.  The slices of a
        # split product of this arrangement meet through scratch memory and tickets, which costs
        # far more than the idle SMs of few tiles (q/k/v of the 7B shape at 130 to 512 tokens:
        # 57 to 93 us split in 2 to 4, 25 to 27 us whole); slices that add into a float32 output
        # with red.add are the cheaper ones there (o_proj 26 against 36 us, down 50 against 110 us).
        splits = 1
    cluster = bool(swap and CLUSTER_SPLITS and 2 <= splits <= 8)
    if cluster and accumulate and M <= RED_MAX_TOKENS and (K + 63) // 64 <= RED_MAX_K_BLOCKS:
        # few tokens, few tiles, added into float32: the slices add their shares with red.add
        tiles = (N + 127) // 128
        if tiles * splits * 2 <= sms():
            cluster, splits = False, _ticket_splits(tiles, (K + 63) // 64, bn)
    tall = tall_tiles(M, N, swap, bn, splits, K, bool(accumulate))
    if tall:
        bn = tall
    if splits == 1 and (wide or pair_tiles(M, N, swap, bn)):
        tall, bn = 2, pair_tile_width(M, N)
    elif accumulate and splits > 1 and PAIR_SPLIT_K and pair_tiles(M, N, swap, bn) and pair_splits(M, N, K) > 1:
        # few tiles, added into float32: slices of K on pairs of SMs (see pair_splits)
        tall, bn, splits = 2, 256, pair_splits(M, N, K)
    scratch, counters, status = workspace(x.device)
    if swap:
        a, b = w, x
    else:
        a, b = x, w
    _check("gemm_tc", library().wpc_gemm_tc(
        _p(a), a.stride(0), a.shape[0], _p(b), b.stride(0), b.shape[0], K, _p(bias), _p(out), _code(out.dtype),
        out.stride(0), accumulate, 0, int(swap), bn, splits, _p(scratch), ctypes.c_size_t(scratch.numel()),
        _p(counters), counters.numel(), _p(status), int(static_weight), (2 if tall == 2 else int(bool(tall))),
        int(cluster), _stream()))
    return True


ACTIVATIONS = {"silu": 1, "gelu_tanh": 2}     # the codes WPC_ACT_* of csrc/common.cuh


def _act(name: str) -> int:
    try:
        return ACTIVATIONS[name]
    except KeyError:
        raise KernelError(f"unknown activation {name!r}; the kernels know {sorted(ACTIVATIONS)}") from None


def gate_mul(gu: torch.Tensor, inner: int, group: Optional[int] = None, activation: str = "silu") -> torch.Tensor:
    """act(gate) * up, where a row of gu holds gate and up interleaved in blocks of `group`
    features ([group gates | group ups | ...]); group None or inner: all gates, then all ups.
    activation: "silu" (g / (1 + exp(-g))) or "gelu_tanh"."""
    group = inner if group is None else group
    _need(gu.is_contiguous() and gu.dim() == 2 and gu.shape[1] == 2 * inner, "gu must be contiguous [T, 2*inner]")
    _need(group >= 1 and inner % group == 0, "group must divide inner")
    out = torch.empty((gu.shape[0], inner), dtype=gu.dtype, device=gu.device)
    _check("gate_mul", library().wpc_gate_mul(_p(gu), _p(out), _code(gu.dtype), gu.shape[0], inner, group,
                                              _act(activation), _stream()))
    return out


def silu_mul(gu: torch.Tensor, inner: int, group: Optional[int] = None) -> torch.Tensor:
    """silu(gate) * up: `gate_mul` with the reference's activation (model.rs:527-531)."""
    return gate_mul(gu, inner, group, "silu")


GATED_GROUP = 64      # gate/up interleave that lets the tensor-core product apply silu(gate) * up itself


def gated_linear(x: torch.Tensor, w: torch.Tensor, inner: int, group: int, plain: bool = False,
                 static_weight: bool = False, activation: str = "silu") -> torch.Tensor:
    """act(x Wg^T) * (x Wu^T) as [T, inner], where w [2*inner, K] holds the rows of Wg and Wu
    interleaved in blocks of `group`.  With bfloat16 and group 64 the tensor-core product
    applies the activation in its epilogue and the [T, 2*inner] intermediate never reaches
    memory; otherwise a product and `gate_mul` follow one another."""
    act = _act(activation)
    _rows(x, "x")
    _rows(w, "w")
    M, K = x.shape
    _need(w.shape == (2 * inner, K), "w must be [2*inner, K]")
    if (not plain and group == GATED_GROUP and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
            and K % 8 == 0 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0
            and w.data_ptr() % 16 == 0 and M > 0):
        swap = M <= 128
        bn = (16 if M <= 16 else 32 if M <= 32 else 64 if M <= 64 else 128) if swap else (256 if (2 * inner) % 256 == 0 else 128)
        tall = tall_tiles(M, 2 * inner, swap, bn, 1) == 256      # the gated epilogue needs whole 128-column groups
        if pair_tiles(M, 2 * inner, swap, bn, padded=False):
            tall = 2
        if swap and bn == 128 and (2 * inner) % 256 == 0:
            # 65..128 tokens: every SM takes in the token tile once for 256 weight rows instead of
            # twice (gate/up of the 7B shape at 128 tokens: 69.5 against 74.6 us; with 64 tokens
            # and less, two narrow tiles to an SM stream better: 53.8 against 63.2 us)
            tall = 1
        # few tokens and fewer tiles than SMs (a small model): K is split over clusters, as in linear()
        splits = 1
        tiles, k_blocks = (2 * inner + 127) // 128, (K + 63) // 64
        if swap and CLUSTER_SPLITS and not tall and tiles < sms():
            for s in range(min(8, k_blocks // 4), 1, -1):
                if tiles <= cluster_capacity(bn, s) and tiles * s <= 2 * sms():
                    splits = s
                    break
        out = torch.empty((M, inner), dtype=torch.bfloat16, device=x.device)
        scratch, counters, status = workspace(x.device)
        a, b = (w, x) if swap else (x, w)
        _check("gemm_tc", library().wpc_gemm_tc(
            _p(a), a.stride(0), a.shape[0], _p(b), b.stride(0), b.shape[0], K, _p(None), _p(out), _BF16,
            out.stride(0), 0, act, int(swap), bn, splits, _p(scratch), ctypes.c_size_t(scratch.numel()), _p(counters),
            counters.numel(), _p(status), int(static_weight), int(tall), int(splits > 1), _stream()))
        return out
    return gate_mul(linear(x, w, plain=plain, static_weight=static_weight), inner, group, activation)


def add_(x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
    """x += y in float32, in place (x float32)."""
    _need(x.dtype == torch.float32 and x.is_contiguous() and y.is_contiguous() and x.shape == y.shape,
          "x must be contiguous float32 and y of the same shape")
    _check("add", library().wpc_add(_p(x), _p(y), _code(y.dtype), ctypes.c_size_t(x.numel()), _stream()))
    return x


def gather_rows(x: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
    _need(x.dtype == torch.float32 and x.is_contiguous() and idx.dtype == torch.int32, "x float32, idx int32")
    out = torch.empty((idx.numel(), x.shape[1]), dtype=torch.float32, device=x.device)
    _check("gather_rows", library().wpc_gather_rows(_p(x), _p(idx), _p(out), idx.numel(), x.shape[1], x.shape[0],
                                                    _stream()))
    return out


def convert(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    if x.dtype == dtype:
        return x
    _need(x.is_contiguous(), "x must be contiguous")
    out = torch.empty(x.shape, dtype=dtype, device=x.device)
    _check("convert", library().wpc_convert(_p(x), _code(x.dtype), _p(out), _code(dtype),
                                            ctypes.c_size_t(x.numel()), _stream()))
    return out


def rope_angles(positions: torch.Tensor, inv_freq: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """cos and sin, float32 [T, R], of positions[t] * inv_freq[r] computed in float64."""
    _need(positions.dtype == torch.int32 and inv_freq.dtype == torch.float64, "positions int32, inv_freq float64")
    T, R = positions.numel(), inv_freq.numel()
    cos = torch.empty((T, R), dtype=torch.float32, device=positions.device)
    sin = torch.empty_like(cos)
    _check("rope_angles", library().wpc_rope_angles(_p(positions), _p(inv_freq), _p(cos), _p(sin), T, R, _stream()))
    return cos, sin


def rope_inplace(x: torch.Tensor, n_heads: int, head_dim: int, cos: torch.Tensor, sin: torch.Tensor,
                 interleaved: bool = False) -> torch.Tensor:
    """Rotates the first n_heads heads of every row of x in place: pair r of a head is the
    elements (r, r + head_dim/2) (rope.rs:34-37), or (2r, 2r + 1) with `interleaved`."""
    _rows(x, "x")
    _need(x.shape[1] >= n_heads * head_dim and cos.shape == sin.shape and cos.shape[0] == x.shape[0],
          "x too narrow or tables of the wrong length")
    _need(cos.dtype == torch.float32 and cos.is_contiguous() and sin.is_contiguous(), "tables: contiguous float32")
    _check("rope_inplace", library().wpc_rope_inplace(_p(x), _code(x.dtype), x.stride(0), x.shape[0], n_heads,
                                                      head_dim, cos.shape[1], _p(cos), _p(sin), int(bool(interleaved)),
                                                      _stream()))
    return x


def head_rmsnorm_(x: torch.Tensor, n_heads: int, head_dim: int, gain: torch.Tensor, eps: float) -> torch.Tensor:
    """RMS norm with gain [head_dim] of each of the first n_heads heads of every row of x, in
    place (the per-head q/k norm of wpc-runtime/src/model.rs:447-462)."""
    _rows(x, "x")
    _need(x.shape[1] >= n_heads * head_dim, "x is too narrow")
    _need(gain.dtype == torch.float32 and gain.numel() == head_dim and gain.is_contiguous(), "gain: float32 [head_dim]")
    _check("head_rmsnorm", library().wpc_head_rmsnorm(_p(x), _code(x.dtype), x.stride(0), x.shape[0], n_heads, head_dim,
                                                      _p(gain), ctypes.c_float(eps), _stream()))
    return x


def qk_rope_kv_store(qkv: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int,
                     cos: Optional[torch.Tensor], sin: Optional[torch.Tensor],
                     k_pages: torch.Tensor, v_pages: torch.Tensor, page_table: torch.Tensor,
                     seq_of_token: torch.Tensor, positions: torch.Tensor) -> None:
    """Rotates q and k of qkv [T, (n_heads + 2 n_kv_heads) head_dim] (q in place) and appends
    the rotated k and the v of every token to the pages of its sequence."""
    _rows(qkv, "qkv")
    _need(qkv.shape[1] == (n_heads + 2 * n_kv_heads) * head_dim, "qkv has the wrong width")
    _need(k_pages.is_contiguous() and v_pages.is_contiguous() and k_pages.dtype == qkv.dtype
          and tuple(k_pages.shape[1:]) == (n_kv_heads, PAGE, head_dim) and k_pages.shape == v_pages.shape,
          "pages must be contiguous [n_pages, n_kv_heads, PAGE, head_dim] of qkv's type")
    _need(page_table.dtype == torch.int32 and page_table.is_contiguous(), "page_table must be contiguous int32")
    R = 0 if cos is None else cos.shape[1]
    _, _, status = workspace(qkv.device)
    _check("qk_rope_kv_store", library().wpc_qk_rope_kv_store(
        _p(qkv), _code(qkv.dtype), qkv.stride(0), qkv.shape[0], n_heads, n_kv_heads, head_dim, R, _p(cos), _p(sin),
        _p(k_pages), _p(v_pages), _p(page_table), page_table.shape[1], _p(seq_of_token), _p(positions),
        k_pages.shape[0], _p(status), _stream()))


PREFILL_ATTENTION_TILES = 1     # row tiles of 128 rows to a CTA of the tcgen05 prefill attention (1 or 2)
FUSE_ROPE_STORE = True     # the q/k/v product rotates and writes the cache itself (cluster tail, pair epilogue)


def linear_qk_rope_kv_store(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], n_heads: int,
                            n_kv_heads: int, head_dim: int, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor],
                            k_pages: torch.Tensor, v_pages: torch.Tensor, page_table: torch.Tensor,
                            seq_of_token: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
    """qkv = x w^T + bias with q and k rotated and k, v appended to the cache: `linear`
    followed by `qk_rope_kv_store`, or, with few tokens in bfloat16, one kernel that does the
    rotation and the cache write in the product's tail (csrc/gemm_tc.cu).  Only the q columns
    of the result are meant to be read."""
    M, K = x.shape
    N = w.shape[0]
    if (FUSE_ROPE_STORE and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and k_pages.dtype == torch.bfloat16
            and head_dim in (16, 32, 64, 128) and M > 0 and N == (n_heads + 2 * n_kv_heads) * head_dim
            and K % 8 == 0 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0
            and w.data_ptr() % 16 == 0 and x.stride(1) == 1 and w.stride(1) == 1):
        swap, bn, splits = plan_tensor_core_linear(M, N, K)
        few = swap and CLUSTER_SPLITS and 2 <= splits <= 8                  # the cluster variant's tail
        many = (not swap) and head_dim >= 64 and pair_tiles(M, N, swap, bn)   # the pair kernel's epilogue (K whole: see _tensor_core_linear)
        if few or many:
            if many:
                bn = 256
            _need(k_pages.is_contiguous() and v_pages.is_contiguous() and k_pages.shape == v_pages.shape
                  and tuple(k_pages.shape[1:]) == (n_kv_heads, PAGE, head_dim),
                  "pages must be contiguous [n_pages, n_kv_heads, PAGE, head_dim]")
            _need(page_table.dtype == torch.int32 and page_table.is_contiguous(), "page_table must be contiguous int32")
            if bias is not None:
                _need(bias.dtype == torch.float32 and bias.numel() == N and bias.is_contiguous(), "bias must be float32 [N]")
            R = 0 if cos is None else cos.shape[1]
            out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
            _, _, status = workspace(x.device)
            _check("gemm_tc_rope_store", library().wpc_gemm_tc_rope_store(
                _p(w), w.stride(0), _p(x), x.stride(0), M, K, _p(bias), _p(out), out.stride(0), bn, splits, 1,
                n_heads, n_kv_heads, head_dim, R, _p(cos), _p(sin), _p(k_pages), _p(v_pages), _p(page_table),
                page_table.shape[1], _p(seq_of_token), _p(positions), k_pages.shape[0], _p(status), _stream()))
            return out
    qkv = linear(x, w, bias, static_weight=True)
    qk_rope_kv_store(qkv, n_heads, n_kv_heads, head_dim, cos, sin, k_pages, v_pages, page_table, seq_of_token, positions)
    return qkv


def attention(q: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int, k_pages: torch.Tensor,
              v_pages: torch.Tensor, page_table: torch.Tensor, cu_seqlens: torch.Tensor, ctx_lens: torch.Tensor,
              seq_of_token: torch.Tensor, positions: torch.Tensor, scale: float, window: Optional[int],
              max_new_tokens: int, max_ctx_len: int, splits: Optional[int] = None,
              mma_only: bool = False, cluster: Optional[int] = None, groups: int = 1) -> torch.Tensor:
    """softmax(q . k * scale) . v over the cached positions that each query sees: 0..its own,
    or the last `window` of them.  q: the first n_heads*head_dim columns of each row.

    bfloat16 with a head size that is a multiple of 16 up to 128 runs on the tensor cores: the
    split-KV kernel when every sequence brings one token (csrc/attention_mma.cu; `splits` forces
    about that many CTAs to a pair, `cluster` `groups` clusters of that size to a pair, 0 none); otherwise the
    tcgen05 kernel for head sizes 64 and 128 (csrc/attention_tc.cu) and the mma.sync kernel for
    the others (or with `mma_only`).  Everything else runs the plain kernel."""
    if q.dtype != torch.bfloat16 or not library().wpc_attention_mma_supports(n_heads, n_kv_heads, head_dim):
        return attention_plain(q, n_heads, n_kv_heads, head_dim, k_pages, v_pages, page_table, seq_of_token,
                               positions, scale, window, max_ctx_len)
    _rows(q, "q")
    _need(q.shape[1] >= n_heads * head_dim, "q is too narrow")
    _need(k_pages.is_contiguous() and v_pages.is_contiguous() and k_pages.dtype == q.dtype, "pages: wrong type")
    T, B = q.shape[0], ctx_lens.numel()
    out = torch.empty((T, n_heads * head_dim), dtype=q.dtype, device=q.device)
    if max_new_tokens == 1 and B <= 1024 and B * n_kv_heads <= _WORKSPACE_COUNTERS:
        _need(T == B, "one token per sequence expected")
        if cluster is None:
            cluster, groups = (0, 1) if splits else plan_decode_cluster(B, n_kv_heads, n_heads, head_dim,
                                                                        max_ctx_len, window)
        if cluster:
            part_o = part_ml = counters = None
            if groups > 1:
                pairs = B * n_kv_heads
                part_o = torch.empty((pairs * groups * (n_heads // n_kv_heads) * head_dim,), dtype=torch.float32,
                                     device=q.device)
                part_ml = torch.empty((pairs * groups * 32,), dtype=torch.float32, device=q.device)
                _, counters, _ = workspace(q.device)
            _check("attention_decode_cluster", library().wpc_attention_decode_cluster(
                _p(q), q.stride(0), _p(out), out.stride(0), _p(k_pages), _p(v_pages), _p(page_table),
                page_table.shape[1], _p(ctx_lens), B, n_heads, n_kv_heads, head_dim, ctypes.c_float(scale),
                int(window or 0), int(cluster), int(groups), _p(part_o), _p(part_ml), _p(counters),
                0 if counters is None else counters.numel(), _stream()))
            return out
        n_ctas = plan_decode_ctas(B, n_kv_heads, max_ctx_len, window, splits)
        slots = n_ctas + B * n_kv_heads
        part_o = torch.empty((slots * 16 * head_dim,), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((slots * 16 * 2,), dtype=torch.float32, device=q.device)
        _, counters, _ = workspace(q.device)
        _check("attention_decode", library().wpc_attention_decode(
            _p(q), q.stride(0), _p(out), out.stride(0), _p(k_pages), _p(v_pages), _p(page_table),
            page_table.shape[1], _p(ctx_lens), B, n_heads, n_kv_heads, head_dim, ctypes.c_float(scale),
            int(window or 0), n_ctas, _p(part_o), _p(part_ml), _p(counters), counters.numel(), _stream()))
    elif (not mma_only and library().wpc_attention_prefill_tc_supports(n_heads, n_kv_heads, head_dim)
          and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0):
        _, _, status = workspace(q.device)
        _check("attention_prefill_tc", library().wpc_attention_prefill_tc(
            _p(q), q.stride(0), _p(out), out.stride(0), _p(k_pages), _p(v_pages), _p(page_table),
            page_table.shape[1], _p(cu_seqlens), _p(ctx_lens), B, max_new_tokens, n_heads, n_kv_heads, head_dim,
            ctypes.c_float(scale), int(window or 0), _p(status), k_pages.shape[0], PREFILL_ATTENTION_TILES,
            _stream()))
    else:
        _check("attention_prefill", library().wpc_attention_prefill(
            _p(q), q.stride(0), _p(out), out.stride(0), _p(k_pages), _p(v_pages), _p(page_table),
            page_table.shape[1], _p(cu_seqlens), _p(ctx_lens), B, max_new_tokens, n_heads, n_kv_heads, head_dim,
            ctypes.c_float(scale), int(window or 0), _stream()))
    return out


def plan_decode_ctas(n_seqs: int, n_kv_heads: int, max_ctx_len: int, window: Optional[int],
                     per_pair: Optional[int] = None) -> int:
    """How many CTAs share the pages of a decode step on the fixed grid (see _plan_decode)."""
    return _plan_decode(n_seqs, n_kv_heads, max_ctx_len, window, per_pair)[0]


def _plan_decode(n_seqs: int, n_kv_heads: int, max_ctx_len: int, window: Optional[int],
                 per_pair: Optional[int] = None):
    """(CTAs, estimated microseconds) for the pages of a decode step on the fixed grid: two CTAs
    to an SM (an SM takes in only so many bytes a second, so all of them should stream), fewer
    when there are not even four pages of work for each.  `per_pair` forces about that many
    CTAs per (sequence, kv head)."""
    blocks = (max_ctx_len + PAGE - 1) // PAGE
    if window:
        blocks = min(blocks, (window + PAGE - 1) // PAGE + 1)
    pairs = max(n_seqs * n_kv_heads, 1)
    if per_pair:
        return max(1, min(pairs * per_pair, 1024)), 0.0
    if 3 * sms() // 2 <= pairs <= 2 * sms():
        # nearly two pairs to an SM: a CTA to a pair, so that equally long sequences need no
        # combining at all (64 sequences x 4 KV heads of 4,000 positions: 91 against 99 us);
        # with fewer pairs than that, fewer CTAs would stream too little (192 CTAs: 90 against 77 us)
        return pairs, 2.0 + 1.5 * blocks
    # Otherwise the count with the least estimated time (microseconds, fitted to measurements at
    # the 7B shape: a page takes a CTA 1.05 us when it has an SM and a deep ring to itself, 1.5 us
    # when two share an SM and its bandwidth, which also costs about 2 us at the start; combining
    # the parts of a pair costs about 7 + 0.12 per part: partial results to L2, a ticket, and the
    # last CTA's pass over all parts, 1.1 + 5.0 us with 8 parts, behind the slowest CTA's pages).  When all sequences are about equally long, a share of pages that
    # divides a pair's pages keeps every CTA inside one pair; a CTA that straddles two pairs
    # fills its ring, merges and takes a ticket twice (about 8 us).  One sequence of 4,000
    # positions: 84 CTAs of 3 pages, 14 us, against 60 CTAs of 4 or 5 pages, 18 us.
    def estimate(n, per, aligned):
        page, start = (1.05, 0.0) if n <= sms() else (1.5, 2.0)
        parts = -(-blocks // per)
        return start + per * page + (7.0 + 0.12 * parts if parts > 1 else 0.0) + (0.0 if aligned else 8.0) + 0.002 * n

    units = pairs * blocks
    target = max(1, min(2 * sms(), pairs * max(blocks // 4, 1)))
    best_n, best_t = target, estimate(target, -(-units // target), False)
    for per in range(1, blocks + 1):
        if blocks % per == 0:
            n = pairs * (blocks // per)
            if n <= 2 * sms():
                t = estimate(n, per, True)
                if t < best_t:
                    best_n, best_t = n, t
    return best_n, best_t


# Decode attention with a thread-block cluster to each (sequence, kv head) pair (see
# csrc/attention_mma.cu): on, and the sizes it takes.
CLUSTER_DECODE = True
CLUSTER_DECODE_MAX_OUT = 1024
_decode_cluster_capacity: dict = {}


def decode_cluster_capacity(head_dim: int, cluster: int, alone: bool) -> int:
    """Clusters of `cluster` CTAs of the cluster decode kernel that this device runs at once
    (a cluster lives inside one GPC, and chips differ in the SMs that their GPCs have)."""
    key = (head_dim, cluster, alone)
    if key not in _decode_cluster_capacity:
        _decode_cluster_capacity[key] = max(0, int(library().wpc_attention_decode_cluster_capacity(
            head_dim, cluster, int(alone))))
    return _decode_cluster_capacity[key]


# Microseconds of the cluster decode kernel, fitted to runs at the 7B shape (1 to 6 sequences of
# 8 Ki to 64 Ki positions, every cluster size and group count that fits; root mean square error
# 0.9 us): a page when a CTA has an SM to itself and when two share one, what sharing costs at
# the start, the exchange through shared memory, and what several groups to a pair add (parts to
# L2, a fence, a ticket, a cluster barrier, one pass over the parts) with so much more a group.
CLUSTER_PAGE_ALONE_US, CLUSTER_PAGE_SHARED_US, CLUSTER_SHARED_START_US = 0.97, 1.29, 1.0
CLUSTER_EXCHANGE_US, GROUP_COMBINE_US, GROUP_EACH_US = 4.1, 3.3, 0.23


def plan_decode_cluster(n_seqs: int, n_kv_heads: int, n_heads: int, head_dim: int, max_ctx_len: int,
                        window: Optional[int]):
    """(cluster size 2..16, groups) if a decode step should run with clusters to a pair, else
    (0, 1): whichever the estimates make fastest, the fixed grid's being that of plan_decode_ctas
    (at the 7B shape, 8 sequences of 4,000 positions: clusters of 7 take 20.3 us, 256 CTAs with
    tickets 24.8).  Every pair gets the
    same number of CTAs and all clusters must run at once, with a tenth of the device's
    capacity to spare: clusters are placed while CTAs of the kernel before still hold their
    SMs, and one that finds no room in any GPC waits for the others to end (32 clusters of 8
    where 33 fit: 28 to 32 us in most launches, 18 us in the others).  When 16 ranks to a pair
    leave SMs idle (one or two long sequences), several clusters (groups) share a pair's pages
    and the pair's last cluster adds their parts (one sequence of 32 Ki positions: 7 groups of 8,
    21.7 us; the fixed grid 28.5, one cluster of 16 35)."""
    pairs = max(n_seqs * n_kv_heads, 1)
    if not CLUSTER_DECODE or (n_heads // n_kv_heads) * head_dim > CLUSTER_DECODE_MAX_OUT or pairs > sms():
        return 0, 1
    blocks = (max_ctx_len + PAGE - 1) // PAGE
    if window:
        blocks = min(blocks, (window + PAGE - 1) // PAGE + 1)
    best, best_t = (0, 1), _plan_decode(n_seqs, n_kv_heads, max_ctx_len, window)[1]
    for c in range(2, 17):
        for g in range(1, 17):
            n = pairs * c * g
            if n > 2 * sms() or c * g > blocks:
                break
            if g > 1 and c < 4:
                continue                    # small clusters in groups: larger clusters do the same with less combining
            alone = n <= sms()
            if pairs * g * 1.1 > decode_cluster_capacity(head_dim, c, alone):
                continue                    # more groups may fit again once two CTAs share an SM
            page, start = ((CLUSTER_PAGE_ALONE_US, 0.0) if alone else
                           (CLUSTER_PAGE_SHARED_US, CLUSTER_SHARED_START_US))
            t = (start + -(-blocks // (c * g)) * page + CLUSTER_EXCHANGE_US +
                 (GROUP_COMBINE_US + GROUP_EACH_US * g if g > 1 else 0.0))
            if t < best_t:
                best, best_t = (c, g), t
    return best


def attention_plain(q, n_heads, n_kv_heads, head_dim, k_pages, v_pages, page_table, seq_of_token, positions,
                    scale, window, max_ctx_len: Optional[int] = None, splits: Optional[int] = None) -> torch.Tensor:
    """The attention of the 32-bit path and the plain twin of the fast kernels: a block to each
    (token, head).  With few tokens and long contexts (`max_ctx_len`, the longest sequence of
    the step) several blocks share a query's keys, about 256 each and no more blocks than fill
    the device twice (`splits` forces their number); their parts are added in order."""
    _rows(q, "q")
    _need(q.shape[1] >= n_heads * head_dim, "q is too narrow")
    _need(k_pages.is_contiguous() and v_pages.is_contiguous() and k_pages.dtype == q.dtype, "pages: wrong type")
    T = q.shape[0]
    out = torch.empty((T, n_heads * head_dim), dtype=q.dtype, device=q.device)
    if splits is None:
        keys = min(max_ctx_len or 0, window or (max_ctx_len or 0))
        splits = max(1, min(keys // 256, 2 * sms() // max(T * n_heads, 1)))
    part = None
    if splits > 1:
        part = torch.empty((T * n_heads * splits * (head_dim + 2),), dtype=torch.float32, device=q.device)
    _check("attention_plain", library().wpc_attention_plain(
        _p(q), q.stride(0), _p(out), out.stride(0), _code(q.dtype), _p(k_pages), _p(v_pages), _p(page_table),
        page_table.shape[1], _p(seq_of_token), _p(positions), T, n_heads, n_kv_heads, head_dim,
        ctypes.c_float(scale), int(window or 0), int(splits), _p(part), _stream()))
    return out


def sample(logits: torch.Tensor, slots: torch.Tensor, seq_state: torch.Tensor, temperature: float,
           banned: Optional[torch.Tensor]) -> torch.Tensor:
    """One token per row (int32).  temperature 0: the first greatest logit; else a draw from
    softmax(logits / temperature) with the uniform number that the row's state names
    (seq_state[slot] = position, seed, request number, tokens drawn; the last is advanced)."""
    _need(logits.dtype == torch.float32 and logits.is_contiguous() and logits.dim() == 2, "logits: float32 [B, V]")
    _need(slots.dtype == torch.int32 and slots.numel() == logits.shape[0], "slots: int32 [B]")
    _need(seq_state.dtype == torch.int64 and seq_state.is_contiguous() and seq_state.shape[1] == 4,
          "seq_state: int64 [n_slots, 4]")
    out = torch.empty((logits.shape[0],), dtype=torch.int32, device=logits.device)
    nb = 0 if banned is None else banned.numel()
    _check("sample", library().wpc_sample(_p(logits), logits.shape[0], logits.shape[1], _p(slots), _p(seq_state),
                                          ctypes.c_float(temperature), _p(banned), nb, _p(out), _stream()))
    return out


def fill_normal(t: torch.Tensor, key: int, mean: float, std: float) -> None:
    _need(t.is_contiguous(), "t must be contiguous")
    _check("fill_normal", library().wpc_fill_normal(_p(t), _code(t.dtype), ctypes.c_size_t(t.numel()),
                                                    ctypes.c_uint64(key), ctypes.c_float(mean), ctypes.c_float(std),
                                                    _stream()))
