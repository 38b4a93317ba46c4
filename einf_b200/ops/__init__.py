"""Python entry points of the hand-written sm_100a kernels.

Every function takes CUDA tensors, checks what the kernel assumes (dtype,
contiguity, the sizes it can take) and launches on the current stream.  There
is no other backend: a tensor that is not on a CUDA device, a size a kernel
cannot take, or a kernel library that cannot be built raises an error.

The plain PyTorch statement of each function lives beside the tests
(``tests/kernel_references.py``), where it is compared with the kernel.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

from . import _library
from ._library import KernelLibraryError, ensure_built

FLOAT32, BFLOAT16 = 0, 1
_DTYPE_CODES = {torch.float32: FLOAT32, torch.bfloat16: BFLOAT16}

STATUS_BAD_TOKEN = 1
STATUS_BAD_PAGE = 2
STATUS_WAIT_EXPIRED = 4

MAX_HEAD_SIZE = 256


class KernelError(RuntimeError):
    """A launch returned a CUDA error."""


class UnsupportedSize(ValueError):
    """A kernel was asked for a size it does not take."""


def _code(t: torch.Tensor) -> int:
    try:
        return _DTYPE_CODES[t.dtype]
    except KeyError:
        raise TypeError(f"kernels take float32 or bfloat16 tensors, got {t.dtype}") from None


def _dev(t: torch.Tensor, name: str) -> int:
    if not t.is_cuda:
        raise KernelError(
            f"{name} is on {t.device}: the kernels run on a CUDA device only and have no CPU path"
        )
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    return t.data_ptr()


def _opt(t: Optional[torch.Tensor], name: str, dtype: torch.dtype) -> int:
    if t is None:
        return 0
    if t.dtype != dtype:
        raise TypeError(f"{name} must be {dtype}, got {t.dtype}")
    return _dev(t, name)


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current stream's handle.  Asked for at every launch, so by the short road where torch
    has one (the public ``current_stream()`` builds an object: 7 us, more than a launch costs)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


_stream_objects: dict[tuple[int, int], "torch.cuda.Stream"] = {}


def current_stream() -> "torch.cuda.Stream":
    """The current stream as an object (for events and synchronisation), cached per handle."""
    if _raw_stream is None:
        return torch.cuda.current_stream()
    device = torch.cuda.current_device()
    handle = _raw_stream(device)
    stream = _stream_objects.get((device, handle))
    if stream is None:
        stream = torch.cuda.current_stream()
        _stream_objects[(device, handle)] = stream
    return stream


#: launches of this package's own kernels since import (library matrix products are not counted)
launch_count = 0


def _check(code: int, what: str) -> None:
    global launch_count
    if code != 0:
        raise KernelError(f"{what}: CUDA error {code}")
    launch_count += 1


_bound: dict[str, object] = {}


def _fn(symbol: str, argtypes, variant: str = ""):
    function = _bound.get((symbol, variant))
    if function is None:
        function = _library.launcher(symbol, argtypes, variant)
        _bound[(symbol, variant)] = function
    return function


# ---------------------------------------------------------------------------
def embed(tokens: torch.Tensor, table: torch.Tensor, residual: torch.Tensor, status: torch.Tensor) -> None:
    """``residual[t] = table[tokens[t]]`` as float; a token outside the table sets the status word."""
    vocab, hidden = table.shape
    if tokens.dtype != torch.int32 or residual.dtype != torch.float32:
        raise TypeError("embed takes int32 tokens and a float32 residual")
    if residual.shape != (tokens.shape[0], hidden):
        raise ValueError(f"residual is {tuple(residual.shape)}, expected {(tokens.shape[0], hidden)}")
    fn = _fn("einf_embed", [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p])
    _check(
        fn(_dev(tokens, "tokens"), _dev(table, "table"), _code(table), _dev(residual, "residual"),
           tokens.shape[0], hidden, vocab, _dev(status, "status"), _stream()),
        "embed",
    )


def add_rmsnorm(
    x: Optional[torch.Tensor],
    residual: torch.Tensor,
    weight: torch.Tensor,
    eps: float,
    out: torch.Tensor,
    rows: Optional[torch.Tensor] = None,
    status: Optional[torch.Tensor] = None,
) -> None:
    """``residual += x`` (summing a leading split dimension of ``x`` if it has one), then
    ``out = weight * residual * rsqrt(mean(residual^2) + eps)``.

    ``x`` may be None.  With ``rows`` (int32 indices), ``out[r]`` is computed from
    row ``rows[r]`` and the residual is not written.  With ``status`` (the step's status word) a
    handful of rows of split-K partial sums may take the kernel that fetches them by TMA, whose
    bounded wait reports there.
    """
    hidden = residual.shape[-1]
    if residual.dtype != torch.float32 or weight.dtype != torch.float32:
        raise TypeError("the residual stream and norm weights are float32")
    if weight.shape != (hidden,):
        raise ValueError(f"norm weight is {tuple(weight.shape)}, expected {(hidden,)}")
    if hidden > 50_000:
        raise UnsupportedSize(f"add_rmsnorm keeps a row in shared memory; width {hidden} > 50000")
    splits, stride, x_code, x_ptr = 1, 0, FLOAT32, 0
    if x is not None:
        if x.dim() == 3:
            splits, stride = x.shape[0], x.shape[1] * x.shape[2]
        if x.shape[-2:] != residual.shape:
            raise ValueError(f"x is {tuple(x.shape)}, residual {tuple(residual.shape)}")
        x_code, x_ptr = _code(x), _dev(x, "x")
    num_rows = rows.shape[0] if rows is not None else residual.shape[0]
    if out.shape != (num_rows, hidden):
        raise ValueError(f"out is {tuple(out.shape)}, expected {(num_rows, hidden)}")
    fn = _fn(
        "einf_add_rmsnorm",
        [c_void_p, c_int, c_int, c_longlong, c_void_p, c_void_p, c_float, c_void_p, c_int, c_void_p,
         c_int, c_int, c_int, c_void_p, c_void_p],
    )
    _check(
        fn(x_ptr, x_code, splits, stride, _dev(residual, "residual"), _dev(weight, "weight"), float(eps),
           _dev(out, "out"), _code(out), _opt(rows, "rows", torch.int32), num_rows, hidden,
           0 if rows is not None else 1, _opt(status, "status", torch.int32), _stream()),
        "add_rmsnorm",
    )


ADVANCE_MAX_GROUPS = 4


def advance_decode(
    token_ids: torch.Tensor,
    positions: torch.Tensor,
    context_lens: torch.Tensor,
    sampled: torch.Tensor,
    slots: list,
    block_tables: list,
    page_size: int,
) -> None:
    """One decode step on, in place, for a step of single tokens: ``token_ids[i] = sampled[i]`` for
    the first ``len(sampled)`` requests, ``positions += 1``, ``context_lens += 1`` and, per cache
    group, ``slots[i] = table[i, position // page] * page + position % page``.  Requests beyond
    ``sampled`` (padding of a graph bucket) and requests that write nothing keep what they have."""
    groups = len(slots)
    if groups > ADVANCE_MAX_GROUPS or groups != len(block_tables):
        raise UnsupportedSize(f"advance_decode takes up to {ADVANCE_MAX_GROUPS} cache groups")
    pointers = []
    for g in range(ADVANCE_MAX_GROUPS):
        if g < groups:
            pointers += [_opt(slots[g], "slots", torch.int32), _opt(block_tables[g], "block_table", torch.int32)]
        else:
            pointers += [0, 0]
    width = block_tables[0].shape[1] if groups else 0
    fn = _fn("einf_advance_decode", [c_void_p] * 4 + [c_int] + [c_void_p] * 8 + [c_int, c_int, c_int, c_void_p])
    _check(
        fn(_opt(token_ids, "token_ids", torch.int32), _opt(positions, "positions", torch.int32),
           _opt(context_lens, "context_lens", torch.int32), _opt(sampled, "sampled", torch.int32), sampled.shape[0],
           *pointers, groups, width, int(page_size), _stream()),
        "advance_decode",
    )


def zero_fresh_state(state: torch.Tensor, state_slots: torch.Tensor, q_start: torch.Tensor,
                     positions: torch.Tensor) -> None:
    """``state[state_slots[r]] = 0`` for every request ``r`` of the step whose first token stands at
    position 0 (``positions[q_start[r]] == 0``); requests without a slot (-1) are skipped.  ``state``
    is ``[slots, ...]`` of any dtype; the index tensors are the step's own inputs, so the launch
    can be captured in a CUDA graph."""
    num_requests = state_slots.shape[0]
    if q_start.shape[0] != num_requests + 1:
        raise ValueError("q_start must hold one more entry than state_slots")
    num_slots = state.shape[0]
    row_bytes = (state.numel() // num_slots) * state.element_size() if num_slots else 0
    fn = _fn("einf_zero_fresh_state", [c_void_p, c_longlong, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p])
    _check(
        fn(_dev(state, "state"), row_bytes, num_slots, _opt(state_slots, "state_slots", torch.int32),
           _opt(q_start, "q_start", torch.int32), _opt(positions, "positions", torch.int32), num_requests, _stream()),
        "zero_fresh_state",
    )


def _maybe_split(x: torch.Tensor, rows: int, width: int, name: str) -> tuple[int, int]:
    """``x`` is ``[rows, width]``, or float32 partial sums ``[splits, rows, width]``: (splits, stride)."""
    if x.dim() == 3:
        if x.dtype != torch.float32 or x.shape[1:] != (rows, width):
            raise ValueError(f"{name}: partial sums must be float32 [splits, {rows}, {width}], got {tuple(x.shape)}")
        return x.shape[0], rows * width
    if x.shape != (rows, width):
        raise ValueError(f"{name} is {tuple(x.shape)}, expected {(rows, width)}")
    return 1, 0


def rope_kv_write(
    qkv: torch.Tensor,
    bias: Optional[torch.Tensor],
    positions: torch.Tensor,
    inv_freq: torch.Tensor,
    slots: Optional[torch.Tensor],
    q_out: torch.Tensor,
    k_cache: Optional[torch.Tensor],
    v_cache: Optional[torch.Tensor],
    num_heads: int,
    num_kv_heads: int,
    head_size: int,
    status: torch.Tensor,
) -> None:
    """Add the QKV bias, rotate Q and K by their positions, write Q to ``q_out`` and
    K, V into the pages at ``slots``.  ``qkv`` is ``[tokens, width]``, or the float32 partial
    sums ``[splits, tokens, width]`` of a split-K product.  Caches are
    ``[pages, kv_heads, page_size, head_size]``; ``slots`` None (with no caches) computes Q only."""
    tokens = qkv.shape[-2]
    width = (num_heads + 2 * num_kv_heads) * head_size
    splits, stride = _maybe_split(qkv, tokens, width, "qkv")
    rotary_dim = 2 * inv_freq.shape[0]
    if rotary_dim > head_size or inv_freq.dtype != torch.float32:
        raise ValueError("inv_freq must be float32 with at most head_size / 2 entries")
    if q_out.numel() != tokens * num_heads * head_size:
        raise ValueError("q_out must hold [tokens, heads, head_size]")
    page_size = num_pages = 0
    k_ptr = v_ptr = 0
    if slots is not None:
        if k_cache is None or v_cache is None:
            raise ValueError("slots given without caches")
        num_pages, kvh, page_size, size = k_cache.shape
        if (kvh, size) != (num_kv_heads, head_size) or v_cache.shape != k_cache.shape:
            raise ValueError(f"cache is {tuple(k_cache.shape)}, expected [pages, {num_kv_heads}, page, {head_size}]")
        if k_cache.dtype != q_out.dtype or v_cache.dtype != q_out.dtype:
            raise TypeError("cache dtype differs from q_out")
        k_ptr, v_ptr = _dev(k_cache, "k_cache"), _dev(v_cache, "v_cache")
    fn = _fn(
        "einf_rope_kv_write",
        [c_void_p, c_int, c_int, c_longlong, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
         c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    )
    _check(
        fn(_dev(qkv, "qkv"), _code(qkv), splits, stride, _code(q_out), _opt(bias, "bias", torch.float32),
           _opt(positions, "positions", torch.int32), _dev(inv_freq, "inv_freq"),
           _opt(slots, "slots", torch.int32), _dev(q_out, "q_out"), k_ptr, v_ptr, tokens, num_heads,
           num_kv_heads, head_size, rotary_dim, page_size, num_pages, _dev(status, "status"), _stream()),
        "rope_kv_write",
    )


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """``out = silu(gate_up[:, :I]) * gate_up[:, I:]``; ``gate_up`` may be float32 partial sums
    ``[splits, tokens, 2 I]`` of a split-K product."""
    tokens, inter = out.shape
    splits, stride = _maybe_split(gate_up, tokens, 2 * inter, "gate_up")
    fn = _fn("einf_silu_mul", [c_void_p, c_int, c_int, c_longlong, c_void_p, c_int, c_longlong, c_int, c_void_p])
    _check(
        fn(_dev(gate_up, "gate_up"), _code(gate_up), splits, stride, _dev(out, "out"), _code(out), tokens, inter,
           _stream()),
        "silu_mul",
    )


def gemm_simt(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor) -> None:
    """``out = x @ weight.T (+ bias)`` with 32-bit FMA accumulation; x rows may be strided."""
    m, k = x.shape
    n = weight.shape[0]
    if weight.shape != (n, k) or out.shape != (m, n):
        raise ValueError(f"gemm: x {tuple(x.shape)}, weight {tuple(weight.shape)}, out {tuple(out.shape)}")
    if x.stride(1) != 1 or out.stride(1) != 1:
        raise ValueError("gemm operands must have unit stride in their last dimension")
    if not (x.is_cuda and out.is_cuda):
        raise KernelError("gemm operands must be on a CUDA device: there is no CPU path")
    fn = _fn(
        "einf_gemm_simt",
        [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_longlong,
         c_longlong, c_void_p],
    )
    _check(
        fn(x.data_ptr(), _code(x), _dev(weight, "weight"), _code(weight), _opt(bias, "bias", torch.float32),
           out.data_ptr(), _code(out), m, n, k, x.stride(0), out.stride(0), _stream()),
        "gemm_simt",
    )


def tcgen05_takes(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """Whether the tensor-core kernel can take these operands (TMA needs 16-byte aligned rows)."""
    return (
        x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.dim() == 2
        and x.stride(1) == 1 and weight.is_contiguous() and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0
        and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0
    )


def gemm_tcgen05_splits(k: int, splits: int) -> int:
    """The number of K ranges a request for ``splits`` really yields (no range is empty)."""
    fn = _fn("einf_gemm_tcgen05_splits", [c_int, c_int])
    return int(fn(k, splits))


def gemm_tcgen05(
    x: torch.Tensor,
    weight: torch.Tensor,
    bias: Optional[torch.Tensor],
    out: torch.Tensor,
    status: torch.Tensor,
    splits: int = 1,
) -> None:
    """``out = x @ weight.T (+ bias)`` on the tcgen05 tensor cores (bfloat16 operands, 32-bit
    accumulation).  ``out`` is ``[tokens, n]`` bfloat16 or float32; with ``splits`` > 1 it is
    float32 ``[splits, tokens, n]`` partial sums over K ranges, which the consumer adds up
    (``splits`` must then be what :func:`gemm_tcgen05_splits` returns)."""
    global launch_count
    tokens, k = x.shape
    n = weight.shape[0]
    if not tcgen05_takes(x, weight):
        raise UnsupportedSize(
            "gemm_tcgen05 takes bfloat16 operands whose rows are 16-byte aligned (K a multiple of 8)"
        )
    if weight.shape != (n, k):
        raise ValueError(f"weight is {tuple(weight.shape)}, expected {(n, k)}")
    if splits > 1:
        if out.dtype != torch.float32 or out.shape != (splits, tokens, n) or not out.is_contiguous():
            raise ValueError(f"split-K output must be contiguous float32 {(splits, tokens, n)}")
        if gemm_tcgen05_splits(k, splits) != splits:
            raise ValueError(f"K = {k} cannot be cut into {splits} non-empty ranges of 64-wide blocks")
        ldo = n
    else:
        if out.shape != (tokens, n) or out.stride(1) != 1:
            raise ValueError(f"out is {tuple(out.shape)}, expected {(tokens, n)}")
        ldo = out.stride(0)
    fn = _fn(
        "einf_gemm_tcgen05",
        [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_longlong, c_longlong, c_int,
         c_void_p, c_void_p],
    )
    if not x.is_cuda:
        raise KernelError("gemm operands must be on a CUDA device: there is no CPU path")
    _check(
        fn(x.data_ptr(), _dev(weight, "weight"), _opt(bias, "bias", torch.float32), out.data_ptr(), _code(out),
           tokens, n, k, x.stride(0), ldo, splits, _dev(status, "status"), _stream()),
        "gemm_tcgen05",
    )


def add_bias(out: torch.Tensor, bias: torch.Tensor) -> None:
    rows, n = out.shape
    fn = _fn("einf_add_bias", [c_void_p, c_int, c_void_p, c_longlong, c_int, c_void_p])
    _check(fn(_dev(out, "out"), _code(out), _opt(bias, "bias", torch.float32), rows, n, _stream()), "add_bias")


def linear(
    x: torch.Tensor,
    weight: torch.Tensor,
    bias: Optional[torch.Tensor],
    out: torch.Tensor,
) -> None:
    """``out = x @ weight.T (+ bias)``.

    bfloat16 activations against a bfloat16 matrix go to the tensor cores through
    the library matrix product (as the reference's ``F.linear`` does,
    ``src/einf/executors/torch/packed_qkv.py:148``); everything else, the whole
    32-bit path included, runs the FMA kernel, which rounds no input.
    """
    if x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.is_contiguous():
        if not x.is_cuda:
            raise KernelError("linear operands must be on a CUDA device: there is no CPU path")
        if out.dtype == torch.bfloat16:
            torch.mm(x, weight.t(), out=out)
        else:
            torch.mm(x, weight.t(), out_dtype=torch.float32, out=out)
        if bias is not None:
            add_bias(out, bias)
        return
    gemm_simt(x, weight, bias, out)


#: up to this many tokens every bfloat16 product runs on this package's tcgen05 kernel with split-K
#: that fills the GPU.  (Measured at 64 tokens, 0.5B sizes, kernel alone: QKV 2.9 against 3.8 us for
#: the library, O 2.7 against 3.3, down 4.3 against 8.8, gate/up 6.3 against 5.9; but with every
#: product cut 14 to 19 ways the consumers add up that many partial sums for 64 rows each, and
#: the step as a whole was slower: 1.63 against 1.57 ms.  See ``TCGEN05_MID_TOKENS``.)
TCGEN05_MAX_TOKENS = 32
#: K is cut at most this many ways: the consumers hold sixteen loads in flight, so up to sixteen partial
#: sums cost them one round trip to L2 and every further batch another (0.5B sizes, decode step at
#: 8 / 16 / 32 tokens: 0.807 / 0.935 / 1.175 ms with 16, 0.839 / 0.958 / 1.227 with 32 / 20 / 10,
#: 0.843 / 1.069 / 1.445 with 8 / 4 / 2).
MAX_SPLITS = 16


#: Between ``TCGEN05_MAX_TOKENS`` and this many tokens the tcgen05 kernel still takes the matrices
#: with few row tiles (at most ``MID_MAX_TILES`` of 128 rows: QKV, O and the down projection of the
#: small models, which as library products are grids of 7 to 9 CTAs), with K cut at most
#: ``MID_MAX_SPLITS`` ways; the gate/up matrix and the output matrix stay with the library.  Measured,
#: whole decode steps of 64 requests at contexts of 1,024 / 4,096 tokens: 0.5B sizes 1.116 -> 1.055 /
#: 1.505 -> 1.443 ms, 1.5B sizes 1.924 -> 1.762 / 2.773 -> 2.620 ms, 7B sizes 4.29 -> 4.15 / 5.85 ->
#: 5.74 ms (2 or 4 ways lose to the library, 16 ways lose to 12: the consumers' many rows).
TCGEN05_MID_TOKENS = 64
MID_MAX_TILES = 40
MID_MAX_SPLITS = 12


def _tcgen05_splits(tokens: int, n: int, k: int) -> int:
    """How many ways to split K, or 0 for the library product."""
    tiles = -(-n // 128)
    if tokens > TCGEN05_MAX_TOKENS:
        if tokens > TCGEN05_MID_TOKENS or tiles > MID_MAX_TILES:
            return 0
        return max(1, min(-(-_sm_count() // tiles), MID_MAX_SPLITS))
    slots = 2 * _sm_count()                     # two CTAs per SM
    fill = -(-slots // tiles)
    # A grid a little larger than one wave is fine while a CTA's share of the weights is small (at
    # 0.5B sizes more, shorter CTAs win: gate/up 4.6 us with 304 CTAs against 5.3 us with 228); when
    # it is hundreds of KB the few CTAs of a second wave cost a whole CTA's time (7B down projection:
    # 308 CTAs of 440 KB), so the grid then stays within the wave.
    if fill > 1 and fill * tiles > slots and 128 * k * 2 // fill > 64 * 1024:
        fill -= 1
    return max(1, min(fill, MAX_SPLITS))


def project(
    x: torch.Tensor,
    weight: torch.Tensor,
    status: torch.Tensor,
    out_dtype: Optional[torch.dtype] = None,
    allow_partial: bool = True,
) -> torch.Tensor:
    """``x @ weight.T`` for a consumer that can add up partial sums.

    Returns ``[tokens, n]`` in ``out_dtype`` (default: x's dtype), or, when the tcgen05 kernel
    splits K to fill the GPU at small token counts, float32 partial sums ``[splits, tokens, n]``
    which :func:`add_rmsnorm`, :func:`rope_kv_write` and :func:`silu_mul` add up themselves.
    """
    tokens, k = x.shape
    n = weight.shape[0]
    out_dtype = out_dtype or x.dtype
    splits = _tcgen05_splits(tokens, n, k) if tcgen05_takes(x, weight) else 0
    if splits and not allow_partial:
        splits = 1
    if splits:
        splits = gemm_tcgen05_splits(k, splits)
        if splits > 1:
            out = torch.empty((splits, tokens, n), dtype=torch.float32, device=x.device)
        else:
            out = torch.empty((tokens, n), dtype=out_dtype, device=x.device)
        gemm_tcgen05(x, weight, None, out, status, splits)
        return out
    out = torch.empty((tokens, n), dtype=out_dtype, device=x.device)
    linear(x, weight, None, out)
    return out


def paged_attention_generic(
    q: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    block_table: torch.Tensor,
    seq_of_token: torch.Tensor,
    positions: torch.Tensor,
    out: torch.Tensor,
    scale: float,
    window: Optional[int],
    status: torch.Tensor,
) -> None:
    """Causal attention of every token of the batch over the pages of its request.

    ``q`` and ``out`` are ``[tokens, heads, head_size]``; caches
    ``[pages, kv_heads, page_size, head_size]``; ``block_table`` ``[requests, width]``
    maps a request's logical page to a physical one.
    """
    tokens, num_heads, head_size = q.shape
    num_pages, num_kv_heads, page_size, size = k_cache.shape
    if size != head_size or v_cache.shape != k_cache.shape:
        raise ValueError("cache head size differs from q")
    if head_size % 8 or head_size > MAX_HEAD_SIZE:
        raise UnsupportedSize(
            f"paged attention takes head sizes that are multiples of 8 up to {MAX_HEAD_SIZE}, got {head_size}"
        )
    if num_heads % num_kv_heads:
        raise UnsupportedSize(f"{num_heads} query heads are not a multiple of {num_kv_heads} key/value heads")
    if not (q.dtype == k_cache.dtype == v_cache.dtype == out.dtype):
        raise TypeError("q, caches and out must share one dtype")
    if out.shape != q.shape:
        raise ValueError("out must have q's shape")
    fn = _fn(
        "einf_paged_attention_generic",
        [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
         c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p],
    )
    _check(
        fn(_dev(q, "q"), _dev(k_cache, "k_cache"), _dev(v_cache, "v_cache"), _code(q),
           _opt(block_table, "block_table", torch.int32), _opt(seq_of_token, "seq_of_token", torch.int32),
           _opt(positions, "positions", torch.int32), _dev(out, "out"), tokens, num_heads, num_kv_heads,
           head_size, page_size, num_pages, block_table.shape[1], float(scale),
           int(window) if window else 0, _dev(status, "status"), _stream()),
        "paged_attention_generic",
    )


#: head sizes the tensor-core attention kernels take (one build per size)
FAST_ATTENTION_MAX_HEAD_SIZE = 128
#: query rows per tile of the prefill attention kernel
Q_TILE = 128


def attention_library(head_size: int) -> str:
    return f"attention_bf16:HEAD_SIZE={head_size}"


def has_tcgen05_attention(head_size: int, page_size: int) -> bool:
    """The tcgen05 prefill kernel is built for head sizes 64 and 128 and pages of 8 to 128 tokens."""
    return head_size in (64, 128) and page_size in (8, 16, 32, 64, 128)


def attention_libraries(head_size: int, page_size: int) -> tuple[str, ...]:
    names = (attention_library(head_size),)
    if has_tcgen05_attention(head_size, page_size):
        names += (f"attention_tcgen05:HEAD_SIZE={head_size}",)
    return names


def has_fast_attention(dtype: torch.dtype, head_size: int) -> bool:
    return dtype == torch.bfloat16 and head_size % 16 == 0 and head_size <= FAST_ATTENTION_MAX_HEAD_SIZE


def _check_fast_attention(q, k_cache, v_cache, out):
    tokens, num_heads, head_size = q.shape
    num_pages, num_kv_heads, page_size, size = k_cache.shape
    if not has_fast_attention(q.dtype, head_size):
        raise UnsupportedSize(
            f"the tensor-core attention kernels take bfloat16 and head sizes in steps of 16 up to "
            f"{FAST_ATTENTION_MAX_HEAD_SIZE}, got {q.dtype} and {head_size}"
        )
    if size != head_size or v_cache.shape != k_cache.shape or out.shape != q.shape:
        raise ValueError("q, caches and out do not fit together")
    if num_heads % num_kv_heads:
        raise UnsupportedSize(f"{num_heads} query heads are not a multiple of {num_kv_heads} key/value heads")
    if not (k_cache.dtype == v_cache.dtype == out.dtype == torch.bfloat16):
        raise TypeError("q, caches and out must be bfloat16")
    return tokens, num_heads, head_size, num_pages, num_kv_heads, page_size


def decode_splits(num_tokens: int, num_heads: int, num_kv_heads: int) -> int:
    """How many ways the keys of one token are split so that a decode launch fills the GPU
    (the reference picks splits per request from its context, qwen.py:40-57; here the kernel
    shortens the splits of a short context itself, so the count depends on the batch only)."""
    head_blocks = (num_heads // num_kv_heads + 15) // 16
    ctas_per_split = max(1, num_tokens * num_kv_heads * head_blocks)
    return max(1, min(16, -(-_sm_count() // ctas_per_split)))


class DecodeWorkspace:
    """Scratch of the split decode kernel: partial outputs, (max, sum) pairs, arrival counters."""

    def __init__(self, tokens: int, num_heads: int, num_kv_heads: int, head_size: int, splits: int, device) -> None:
        self.tokens, self.splits = tokens, splits
        head_blocks = (num_heads // num_kv_heads + 15) // 16
        self.acc = torch.empty((tokens, num_heads, splits, head_size), dtype=torch.float32, device=device)
        self.ml = torch.empty((tokens, num_heads, splits, 2), dtype=torch.float32, device=device)
        self.counters = torch.zeros((tokens, num_kv_heads * head_blocks), dtype=torch.int32, device=device)

    def fits(self, tokens: int, splits: int) -> bool:
        return tokens <= self.tokens and splits <= self.splits


def paged_decode_attention(
    q: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    block_table: torch.Tensor,
    seq_of_token: torch.Tensor,
    positions: torch.Tensor,
    out: torch.Tensor,
    scale: float,
    window: Optional[int],
    workspace: DecodeWorkspace,
    splits: int,
    status: torch.Tensor,
) -> None:
    """Tensor-core attention for tokens that each attend alone (decoding): every token
    attends to the keys of its request up to its own position, split ``splits`` ways."""
    tokens, num_heads, head_size, num_pages, num_kv_heads, page_size = _check_fast_attention(q, k_cache, v_cache, out)
    if not workspace.fits(tokens, splits):
        raise ValueError("the decode workspace is too small for this launch")
    if not 1 <= splits <= 64:
        raise UnsupportedSize(f"decode attention splits a token's keys 1 to 64 ways, not {splits}")
    fn = _fn(
        "einf_paged_decode_attention",
        [c_void_p] * 10 + [c_int] * 6 + [c_float, c_int, c_int, c_void_p, c_void_p],
        f"HEAD_SIZE={head_size}",
    )
    _check(
        fn(_dev(q, "q"), _dev(k_cache, "k_cache"), _dev(v_cache, "v_cache"),
           _opt(block_table, "block_table", torch.int32), _opt(seq_of_token, "seq_of_token", torch.int32),
           _opt(positions, "positions", torch.int32), _dev(out, "out"), workspace.acc.data_ptr(),
           workspace.ml.data_ptr(), workspace.counters.data_ptr(), tokens, num_heads, num_kv_heads, page_size,
           num_pages, block_table.shape[1], float(scale), int(window) if window else 0, splits,
           _dev(status, "status"), _stream()),
        "paged_decode_attention",
    )


def decode_cluster_size(num_tokens: int, num_heads: int, num_kv_heads: int) -> int:
    """CTAs that share one (token, key/value head) in the cluster decode kernel.  Measured on a
    B200 at head size 64: about half the SMs is the sweet spot (more CTAs shorten each CTA's
    key range, but clusters of eight large-shared-memory CTAs are slow to place)."""
    head_blocks = (num_heads // num_kv_heads + 15) // 16
    pairs = max(1, num_tokens * num_kv_heads * head_blocks)
    for cluster in (8, 4, 2):
        if pairs * cluster <= (_sm_count() * 55) // 100:
            return cluster
    return 1


_sm_counts: dict[int, int] = {}


def _sm_count() -> int:
    device = torch.cuda.current_device()
    if device not in _sm_counts:
        _sm_counts[device] = torch.cuda.get_device_properties(device).multi_processor_count
    return _sm_counts[device]


_decode_cluster_room: dict[tuple[int, int, int], int] = {}


def tcgen05_decode_cluster_room(head_size: int, cluster: int) -> int:
    """How many clusters of ``cluster`` CTAs of the tcgen05 decode kernel the device holds at once
    (asked of the CUDA occupancy calculator once per device)."""
    key = (torch.cuda.current_device(), head_size, cluster)
    if key not in _decode_cluster_room:
        fn = _fn("einf_paged_decode_attention_tcgen05_max_clusters", [c_int], f"HEAD_SIZE={head_size}")
        _decode_cluster_room[key] = int(fn(cluster))
    return _decode_cluster_room[key]


def decode_context_bucket(max_context: Optional[int]) -> int:
    """The only thing a decode launch takes from the step's contexts: the longest one, rounded up
    to a power of two from 4,096 on (unknown: 4,096).  Steps whose graphs are kept apart by this
    figure may split their keys differently."""
    bucket = 4096
    while max_context is not None and bucket < max_context:
        bucket *= 2
    return bucket


#: (cluster size, clusters per token) pairs ``decode_plan`` chooses from
DECODE_SHAPES = tuple((c, s) for s in (1, 2, 3, 4, 8) for c in (16, 8, 7, 6, 5, 4, 3, 2, 1))


def decode_plan(num_tokens: int, num_heads: int, num_kv_heads: int, head_size: int, page_size: int,
                max_context: Optional[int] = None) -> tuple[str, int, int]:
    """Which decode kernel serves ``num_tokens`` single tokens, with what cluster size and how
    many clusters per token: ``("tcgen05" | "mma", cluster, splits)``.

    The tcgen05 kernel wherever it takes the sizes (head sizes 64 and 128, pages of 8 to 128
    tokens), the ``mma.sync`` cluster kernel otherwise.  Measured on a B200 (16-token pages): 64
    requests of 4,096 tokens at head size 64 32 us against 50 us; head size 128, 8 requests: 21 us
    against 46 us.

    A token's keys are cut into cluster x splits ranges, one CTA each, all CTAs of the launch on
    the device at once (a grid in two waves costs the kernel twice; at head size 128 one CTA fills
    an SM and the GPCs place fewer clusters of eight than SMs / 8: 16 pairs as clusters of 8 took
    16.9 us, as clusters of 4 about 9).  Among the shapes that fit, the one with the least
    estimated time for the bucket of the longest context (``decode_context_bucket``): a CTA walks
    its 128-key tiles one after the other at 0.9 us each, or at the pace the memory delivers them
    to all CTAs together; a cluster above eight costs 0.6 us more (and 1.7 us more where its CTAs
    share SMs); clusters that meet in global memory cost 3.5 us and 0.2 us for each of them.
    Measured, one request of 32,768 tokens at head size 64 (14 query heads, 2 key/value heads):
    clusters of 8 30.7 us, of 16 17.7 us, four clusters of 16 12.2 us; 8 requests of 32,768
    tokens: 35.7 us as clusters of 8, 28.0 us as four clusters of 4 each; head size 128 (28 and 4
    heads), one request of 32,768 tokens: 32.8 us as clusters of 8, 21.0 us as clusters of 16."""
    key = (torch.cuda.current_device(), num_tokens, num_heads, num_kv_heads, head_size, page_size,
           decode_context_bucket(max_context), DECODE_SHAPES)
    plan = _decode_plans.get(key)
    if plan is None:
        plan = _decode_plans[key] = _plan_decode(num_tokens, num_heads, num_kv_heads, head_size, page_size, key[6])
    return plan


_decode_plans: dict[tuple, tuple[str, int, int]] = {}


def _plan_decode(num_tokens: int, num_heads: int, num_kv_heads: int, head_size: int, page_size: int,
                 context_bucket: int, room=None, sms: Optional[int] = None) -> tuple[str, int, int]:
    """``decode_plan`` without its memory.  ``room(head_size, cluster)`` (how many clusters of a
    size the device holds at once) and ``sms`` are asked of the device unless given: the choice
    itself is plain arithmetic and is tested without a GPU."""
    head_blocks = (num_heads // num_kv_heads + 15) // 16
    pairs = max(1, num_tokens * num_kv_heads * head_blocks)
    if not has_tcgen05_attention(head_size, page_size):
        return "mma", decode_cluster_size(num_tokens, num_heads, num_kv_heads), 1
    tiles = context_bucket // 128
    tile_bytes = 2 * 128 * head_size * 2
    room = room or tcgen05_decode_cluster_room
    sms = sms or _sm_count()
    best, best_us = (1, 1), None
    for cluster, splits in DECODE_SHAPES:
        if pairs * splits > room(head_size, cluster) or pairs * splits > DECODE_SPLIT_SHARES:
            continue
        ctas = pairs * cluster * splits
        per_tile_us = max(0.9, ctas * tile_bytes / 6.5e6)
        us = -(-tiles // (cluster * splits)) * per_tile_us
        us += (0.6 if cluster > 8 else 0.0) + (3.5 + 0.2 * splits if splits > 1 else 0.0)
        if cluster > 8 and ctas > sms:
            us += 1.7       # large clusters that share SMs: 14 pairs of 4,096 tokens 8.6 us as clusters of 16, 8.0 as clusters of 8
        if best_us is None or us < best_us - 1e-9:
            best, best_us = (cluster, splits), us
    return "tcgen05", best[0], best[1]


def paged_decode_attention_auto(
    q: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    block_table: torch.Tensor,
    seq_of_token: torch.Tensor,
    positions: torch.Tensor,
    out: torch.Tensor,
    scale: float,
    window: Optional[int],
    status: torch.Tensor,
    token_list: Optional[torch.Tensor] = None,
    max_context: Optional[int] = None,
) -> None:
    """Decode attention by the kernel, cluster size and number of clusters per token that
    ``decode_plan`` picks for this batch; ``max_context`` is the longest context among the
    tokens (a window shortens it), as the host knows it."""
    tokens = token_list.shape[0] if token_list is not None else q.shape[0]
    if window and max_context is not None:
        max_context = min(max_context, int(window))
    kernel, cluster, splits = decode_plan(tokens, q.shape[1], k_cache.shape[1], q.shape[2], k_cache.shape[2], max_context)
    if kernel == "tcgen05":
        paged_decode_attention_tcgen05(q, k_cache, v_cache, block_table, seq_of_token, positions, out, scale, window,
                                       cluster, status, token_list, splits)
    else:
        paged_decode_attention_cluster(q, k_cache, v_cache, block_table, seq_of_token, positions, out, scale, window,
                                       cluster, status, token_list)


def paged_decode_attention_cluster(
    q: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    block_table: torch.Tensor,
    seq_of_token: torch.Tensor,
    positions: torch.Tensor,
    out: torch.Tensor,
    scale: float,
    window: Optional[int],
    cluster: int,
    status: torch.Tensor,
    token_list: Optional[torch.Tensor] = None,
) -> None:
    """Decode attention whose key splits are the CTAs of a thread-block cluster (1, 2, 4 or 8)
    that merge through distributed shared memory: no scratch in global memory.  With
    ``token_list`` (int32 packed indices) only those tokens are processed."""
    tokens, num_heads, head_size, num_pages, num_kv_heads, page_size = _check_fast_attention(q, k_cache, v_cache, out)
    if token_list is not None:
        tokens = token_list.shape[0]
    if cluster not in (1, 2, 4, 8):
        raise UnsupportedSize(f"the cluster decode kernel takes clusters of 1, 2, 4 or 8 CTAs, not {cluster}")
    fn = _fn(
        "einf_paged_decode_attention_cluster",
        [c_void_p] * 8 + [c_int] * 6 + [c_float, c_int, c_int, c_void_p, c_void_p],
        f"HEAD_SIZE={head_size}",
    )
    _check(
        fn(_dev(q, "q"), _dev(k_cache, "k_cache"), _dev(v_cache, "v_cache"),
           _opt(block_table, "block_table", torch.int32), _opt(seq_of_token, "seq_of_token", torch.int32),
           _opt(positions, "positions", torch.int32), _opt(token_list, "token_list", torch.int32), _dev(out, "out"),
           tokens, num_heads, num_kv_heads, page_size,
           num_pages, block_table.shape[1], float(scale), int(window) if window else 0, cluster,
           _dev(status, "status"), _stream()),
        "paged_decode_attention_cluster",
    )


DECODE_MAX_SPLITS = 8
DECODE_SPLIT_SHARES = 512       # (token, key/value head, head block) pairs x splits of one launch, at most
_decode_split_scratch: dict[str, tuple[torch.Tensor, torch.Tensor]] = {}


def _decode_split_workspace(pairs: int, splits: int, device) -> tuple[torch.Tensor, torch.Tensor]:
    """Where the clusters of a split decode launch meet, per device: their shares (16 heads of up
    to 128 + 2 floats per pair and split) and the arrival counters, which every launch leaves at
    zero.  Launches on one stream run one after the other, so they share it; it is made once and
    never grows, because captured graphs hold its address."""
    if pairs * splits > DECODE_SPLIT_SHARES:
        raise UnsupportedSize(
            f"a split decode launch takes up to {DECODE_SPLIT_SHARES} shares, not {pairs} x {splits}: "
            f"split fewer ways, many tokens fill the device without it"
        )
    key = str(device)
    scratch = _decode_split_scratch.get(key)
    if scratch is None:
        scratch = (
            torch.empty(DECODE_SPLIT_SHARES * 16 * (128 + 2), dtype=torch.float32, device=device),
            torch.zeros(DECODE_SPLIT_SHARES, dtype=torch.int32, device=device),
        )
        _decode_split_scratch[key] = scratch
    return scratch


def paged_decode_attention_tcgen05(
    q: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    block_table: torch.Tensor,
    seq_of_token: torch.Tensor,
    positions: torch.Tensor,
    out: torch.Tensor,
    scale: float,
    window: Optional[int],
    cluster: int,
    status: torch.Tensor,
    token_list: Optional[torch.Tensor] = None,
    splits: int = 1,
) -> None:
    """Decode attention on the tcgen05 tensor cores with the keys as the 128-row operand
    (S^T = K Q^T, O^T = V^T P^T), so the tile is full at any number of query heads.  Key splits
    are the CTAs of a cluster (any size from 1 to 16), as in ``paged_decode_attention_cluster``,
    and, for a few requests with long contexts, ``splits`` such clusters per token whose shares
    the last CTA to finish adds up from global memory; head sizes 64 and 128, pages of 8 to 128
    tokens."""
    tokens, num_heads, head_size, num_pages, num_kv_heads, page_size = _check_fast_attention(q, k_cache, v_cache, out)
    if not has_tcgen05_attention(head_size, page_size):
        raise UnsupportedSize(
            f"the tcgen05 attention kernels take head sizes 64 and 128 and pages of 8 to 128 tokens, "
            f"got {head_size} and {page_size}"
        )
    if token_list is not None:
        tokens = token_list.shape[0]
    if not 1 <= cluster <= 16:
        raise UnsupportedSize(f"the tcgen05 decode kernel takes clusters of 1 to 16 CTAs, not {cluster}")
    if not 1 <= splits <= DECODE_MAX_SPLITS:
        raise UnsupportedSize(f"the tcgen05 decode kernel takes 1 to {DECODE_MAX_SPLITS} clusters per token, not {splits}")
    head_blocks = (num_heads // num_kv_heads + 15) // 16
    shares, counters = (None, None)
    if splits > 1:
        shares, counters = _decode_split_workspace(tokens * num_kv_heads * head_blocks, splits, q.device)
    fn = _fn(
        "einf_paged_decode_attention_tcgen05",
        [c_void_p] * 8 + [c_int] * 6 + [c_float, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p],
        f"HEAD_SIZE={head_size}",
    )
    _check(
        fn(_dev(q, "q"), _dev(k_cache, "k_cache"), _dev(v_cache, "v_cache"),
           _opt(block_table, "block_table", torch.int32), _opt(seq_of_token, "seq_of_token", torch.int32),
           _opt(positions, "positions", torch.int32), _opt(token_list, "token_list", torch.int32), _dev(out, "out"),
           tokens, num_heads, num_kv_heads, page_size,
           num_pages, block_table.shape[1], float(scale), int(window) if window else 0, cluster,
           splits, shares.data_ptr() if splits > 1 else None, counters.data_ptr() if splits > 1 else None,
           _dev(status, "status"), _stream()),
        "paged_decode_attention_tcgen05",
    )


def prefill_prefix_bucket(cached_before: Optional[int]) -> int:
    """The only thing a prefill launch takes from the step's contexts: the largest cluster (8, 4,
    else 1) worth trying for the longest prefix that a prompt portion of the step finds in the
    cache.  Steps with equal buckets launch alike.  A cluster costs a launch about 3 us flat
    (measured: 128 tokens at the start of a prompt 7.9 us alone, 10 to 11 us as any cluster), which
    512 cached tokens repay to clusters of four and 1,024 to clusters of eight."""
    if cached_before is None or cached_before < 512:
        return 1
    return 8 if cached_before >= 1024 else 4


_prefill_cluster_room: dict[tuple[int, int, int], int] = {}


def tcgen05_prefill_cluster_room(head_size: int, cluster: int) -> int:
    """How many clusters of ``cluster`` CTAs of the tcgen05 prefill kernel the device holds at once
    (asked of the CUDA occupancy calculator once per device)."""
    key = (torch.cuda.current_device(), head_size, cluster)
    if key not in _prefill_cluster_room:
        fn = _fn("einf_paged_prefill_attention_tcgen05_max_clusters", [c_int], f"HEAD_SIZE={head_size}")
        _prefill_cluster_room[key] = int(fn(cluster))
    return _prefill_cluster_room[key]


def prefill_cluster_size(ctas: int, head_size: int, cached_before: Optional[int]) -> int:
    """CTAs that share one (row tile, head) of the tcgen05 prefill kernel, each with a run of its
    key tiles: the largest cluster (up to the prefix bucket) of which the device holds ``ctas`` at
    once.  A few row tiles behind a long prefix (a portion of a long prompt) do not fill the GPU,
    and the walk over their keys is a chain of dependent tiles; a grid in two waves costs more than
    the split saves, and so does a split of a portion at the start of its prompt, whose rows see
    few keys.  Measured on a B200, 14 heads of 64, one launch in a chain: 64 tokens after 8,192
    100 us alone, 55 / 32 / 21 us as clusters of 2 / 4 / 8; 512 tokens (56 CTAs) after 4,096 40 us
    alone, 27 as clusters of two, 34 as clusters of four (224 CTAs: two waves); 64 tokens after
    512 12.0 us alone, 9.4 as clusters of four; 256 tokens after none 8.3 us alone, 11.2 as
    clusters of two."""
    for cluster in range(prefill_prefix_bucket(cached_before), 1, -1):
        if ctas <= tcgen05_prefill_cluster_room(head_size, cluster):
            return cluster
    return 1


def paged_prefill_attention(
    q: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    block_table: torch.Tensor,
    q_tiles: torch.Tensor,
    out: torch.Tensor,
    scale: float,
    window: Optional[int],
    status: torch.Tensor,
    use_tcgen05: Optional[bool] = None,
    prefill_cluster: int = 0,
    cached_before: Optional[int] = None,
) -> None:
    """Tensor-core causal attention for prompt portions.  ``q_tiles`` is int32 ``[tiles, 4]``:
    request, first token (packed index), rows (at most ``Q_TILE``), position of the first row.
    Head sizes 64 and 128 with pages of 8 to 128 tokens run the tcgen05 kernel (``use_tcgen05``
    None: whenever it can; measured on a B200, a 2,048-token prompt of 14 heads of size 64 takes
    26 us against 82 us, 28 heads of size 128 take 62 us against 266 us), everything else the
    ``mma.sync`` kernel.  ``prefill_cluster`` (1 to 8; 0: ``prefill_cluster_size`` of the number of
    row tiles and ``cached_before``, the most tokens that a portion of this step finds in the
    cache, if the caller knows it) is the number of CTAs that share a row tile's keys in the
    tcgen05 kernel."""
    tokens, num_heads, head_size, num_pages, num_kv_heads, page_size = _check_fast_attention(q, k_cache, v_cache, out)
    if q_tiles.dtype != torch.int32 or q_tiles.dim() != 2 or q_tiles.shape[1] != 4:
        raise ValueError("q_tiles must be int32 [tiles, 4]")
    can = has_tcgen05_attention(head_size, page_size)
    if use_tcgen05 is None:
        use_tcgen05 = can
    if use_tcgen05:
        if not can:
            raise UnsupportedSize(
                f"the tcgen05 attention kernel takes head sizes 64 and 128 and pages of 8 to 128 tokens, "
                f"got {head_size} and {page_size}"
            )
        fn = _fn(
            "einf_paged_prefill_attention_tcgen05",
            [c_void_p] * 5 + [c_int, c_void_p] + [c_int] * 6 + [c_float, c_int, c_int, c_void_p, c_void_p],
            f"HEAD_SIZE={head_size}",
        )
        cluster = prefill_cluster
        if not cluster:
            if cached_before is not None and window:
                cached_before = min(cached_before, int(window))
            cluster = prefill_cluster_size(num_heads * q_tiles.shape[0], head_size, cached_before)
        _check(
            fn(_dev(q, "q"), _dev(k_cache, "k_cache"), _dev(v_cache, "v_cache"),
               _opt(block_table, "block_table", torch.int32), _dev(q_tiles, "q_tiles"), q_tiles.shape[0],
               _dev(out, "out"), tokens, num_heads, num_kv_heads, page_size, num_pages, block_table.shape[1],
               float(scale), int(window) if window else 0, int(cluster), _dev(status, "status"), _stream()),
            "paged_prefill_attention_tcgen05",
        )
        return
    fn = _fn(
        "einf_paged_prefill_attention",
        [c_void_p] * 5 + [c_int, c_void_p] + [c_int] * 5 + [c_float, c_int, c_void_p, c_void_p],
        f"HEAD_SIZE={head_size}",
    )
    _check(
        fn(_dev(q, "q"), _dev(k_cache, "k_cache"), _dev(v_cache, "v_cache"),
           _opt(block_table, "block_table", torch.int32), _dev(q_tiles, "q_tiles"), q_tiles.shape[0],
           _dev(out, "out"), num_heads, num_kv_heads, page_size, num_pages, block_table.shape[1], float(scale),
           int(window) if window else 0, _dev(status, "status"), _stream()),
        "paged_prefill_attention",
    )


ARGMAX_CHUNKS = 32
_argmax_scratch: dict[str, tuple[torch.Tensor, torch.Tensor, torch.Tensor]] = {}


def _argmax_workspace(rows: int, device) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Partial (value, index) pairs and arrival counters of the two-step argmax, per device;
    launches on one stream run one after the other, so they share it."""
    key = str(device)
    scratch = _argmax_scratch.get(key)
    if scratch is None or scratch[2].shape[0] < rows:
        capacity = max(rows, 64)
        scratch = (
            torch.empty((capacity, ARGMAX_CHUNKS), dtype=torch.float32, device=device),
            torch.empty((capacity, ARGMAX_CHUNKS), dtype=torch.int32, device=device),
            torch.zeros(capacity, dtype=torch.int32, device=device),
        )
        _argmax_scratch[key] = scratch
    return scratch


def argmax(logits: torch.Tensor, tokens: torch.Tensor) -> None:
    """``tokens[r]`` = first index of the largest logit of row ``r``."""
    rows, vocab = logits.shape
    if logits.dtype != torch.float32 or tokens.dtype != torch.int32 or tokens.shape[0] < rows:
        raise TypeError("argmax takes float32 logits and an int32 token buffer")
    values, indices, counters = _argmax_workspace(rows, logits.device)
    fn = _fn("einf_argmax", [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p])
    _check(
        fn(_dev(logits, "logits"), _dev(tokens, "tokens"), rows, vocab, values.data_ptr(), indices.data_ptr(),
           counters.data_ptr(), _stream()),
        "argmax",
    )


def report(tokens: torch.Tensor, count: int, status: torch.Tensor, host: torch.Tensor) -> None:
    """``host[:count] = tokens[:count]; host[count] = status[0]``, written by a kernel into the
    pinned host tensor ``host``; readable after the stream is synchronised."""
    if tokens.dtype != torch.int32 or status.dtype != torch.int32 or host.dtype != torch.int32:
        raise TypeError("report takes int32 tensors")
    if tokens.shape[0] < count or host.shape[0] < count + 1 or not host.is_pinned():
        raise ValueError("report needs count tokens and a pinned host tensor of count + 1 entries")
    fn = _fn("einf_report", [c_void_p, c_int, c_void_p, c_void_p, c_void_p])
    _check(fn(_dev(tokens, "tokens"), count, _dev(status, "status"), host.data_ptr(), _stream()), "report")


def sample(
    logits: torch.Tensor,
    tokens: torch.Tensor,
    temperature: torch.Tensor,
    top_k: torch.Tensor,
    top_p: torch.Tensor,
    min_p: torch.Tensor,
    seed: torch.Tensor,
    sample_index: torch.Tensor,
) -> None:
    """Draw one token per row; rows with temperature 0 take the argmax."""
    rows, vocab = logits.shape
    if logits.dtype != torch.float32 or tokens.dtype != torch.int32 or tokens.shape[0] < rows:
        raise TypeError("sample takes float32 logits and an int32 token buffer")
    if seed.dtype != torch.int64 or sample_index.dtype != torch.int64:
        raise TypeError("seed and sample_index are int64")
    fn = _fn(
        "einf_sample",
        [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
    )
    _check(
        fn(_dev(logits, "logits"), _dev(tokens, "tokens"), rows, vocab,
           _opt(temperature, "temperature", torch.float32), _opt(top_k, "top_k", torch.int32),
           _opt(top_p, "top_p", torch.float32), _opt(min_p, "min_p", torch.float32),
           _dev(seed, "seed"), _dev(sample_index, "sample_index"), _stream()),
        "sample",
    )


__all__ = [
    "KernelError",
    "KernelLibraryError",
    "UnsupportedSize",
    "add_bias",
    "add_rmsnorm",
    "argmax",
    "embed",
    "ensure_built",
    "gemm_simt",
    "gemm_tcgen05",
    "gemm_tcgen05_splits",
    "linear",
    "paged_attention_generic",
    "paged_decode_attention",
    "decode_plan",
    "decode_context_bucket",
    "paged_decode_attention_auto",
    "paged_decode_attention_cluster",
    "paged_decode_attention_tcgen05",
    "paged_prefill_attention",
    "project",
    "rope_kv_write",
    "sample",
    "silu_mul",
    "zero_fresh_state",
]
