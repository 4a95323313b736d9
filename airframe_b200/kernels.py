"""Python face of the CUDA kernel library: one function per C entry point.

Arguments are torch tensors on a CUDA device; each function checks device,
dtype and layout, passes raw pointers and the current stream, and raises
:class:`KernelError` with the library's message when a kernel refuses its
sizes.  Nothing here computes on the host and nothing falls back to torch.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from .csrc import KernelLibraryError, load_library
from .kernels_const import PAGE

F32, BF16 = 0, 1
ACTIVATIONS = {"gelu_tanh": 0, "silu": 1}
PAIRINGS = {"half": 0, "adjacent": 1}
MASKS = {"window": 0, "chunk": 1}      # the last `size` positions / the position's own chunk of `size`
FAST_HEAD_SIZES = (64, 128, 256)       # head sizes that the bfloat16 tensor-core attention kernels take between them


class KernelError(RuntimeError):
    """A kernel refused its arguments or failed to launch."""


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16, got {dtype}")


def _lib():
    return load_library()


def _stream() -> c_void_p:
    # the raw handle of the current stream of the current device (the Stream object of
    # torch.cuda.current_stream() costs several microseconds a call, once per kernel launched)
    return c_void_p(_raw_stream(_current_device()))


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_current_device = getattr(torch._C, "_cuda_getDevice", None)
if _raw_stream is None or _current_device is None:          # an older or newer torch: the documented way
    def _raw_stream(_index):                                 # noqa: F811
        return torch.cuda.current_stream().cuda_stream

    def _current_device():                                   # noqa: F811
        return 0


def _ptr(t, name="tensor", dtype=None, allow_none=False) -> c_void_p:
    if t is None:
        if allow_none:
            return c_void_p(0)
        raise KernelError(f"{name} is required")
    if not t.is_cuda:
        raise KernelError(f"{name} must live on a CUDA device (there is no CPU implementation)")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    return c_void_p(t.data_ptr())


def _rows(t, name) -> int:
    """Row stride in elements of a 2-D tensor whose rows are dense."""
    if t.dim() != 2 or t.stride(1) != 1:
        raise KernelError(f"{name} must be 2-D with dense rows, got shape {tuple(t.shape)} strides {t.stride()}")
    return t.stride(0)


def _check(code: int) -> None:
    if code != 0:
        msg = _lib().af_last_error().decode("utf-8", "replace")
        raise KernelError(f"{msg} (code {code})")


def launch_count() -> int:
    """Kernels this library has launched since it was loaded."""
    f = _lib().af_launch_count
    f.restype = ctypes.c_ulonglong
    return int(f())


def bounds_failures():
    """The checked build's record (see ``csrc.use_checked_build``): None in the
    normal build, else (translation units that saw a bad index since the last
    call, one of the bad values).  Synchronises the device."""
    index = c_int(0)
    n = int(_lib().af_bounds_failures(ctypes.byref(index)))
    if n < 0:
        return None
    return n, int(index.value)


_SMS = {}


def sm_count() -> int:
    """Streaming multiprocessors of the current device (asked of the driver
    once per device): what the policies that cut work into blocks divide by."""
    dev = _current_device()
    n = _SMS.get(dev)
    if n is None:
        n = int(_lib().af_device_sm_count())
        if n <= 0:
            _check(n or -1)
        _SMS[dev] = n
    return n


def require_cuda_tensor(t, name="tensor"):
    if not t.is_cuda:
        raise KernelError(f"{name} must live on a CUDA device")


# ---------------------------------------------------------------- elementwise

def embed(out, table, ids, scale: float) -> None:
    """out[t] = table[ids[t]] * scale; out float32 [T, H]."""
    T, H = out.shape
    _check(_lib().af_embed(_ptr(out, "out", torch.float32), _ptr(table, "table"), c_int(dtype_code(table.dtype)),
                           _ptr(ids, "ids", torch.int32), c_int(T), c_int(H), c_int(table.shape[0]),
                           c_float(scale), _stream()))


def rmsnorm(y, x, w, eps: float, offset: float, rows=None) -> None:
    """y[r] = norm(x[rows[r]] or x[r]) * (offset + w); x, w float32."""
    n, H = y.shape
    if not (x.is_contiguous() and y.is_contiguous()):
        raise KernelError("rmsnorm: tensors must be contiguous")
    _check(_lib().af_rmsnorm(_ptr(y, "y"), c_int(dtype_code(y.dtype)), _ptr(x, "x", torch.float32),
                             _ptr(w, "w", torch.float32), _ptr(rows, "rows", torch.int32, allow_none=True),
                             c_int(n), c_int(H), c_float(eps), c_float(offset), _stream()))


def add_rmsnorm(x, a, w_post, eps_post: float, offset: float, y=None, w_next=None, eps_next: float = 0.0,
                n_parts: int = 1) -> None:
    """x += norm(a) * (offset + w_post); if y: y = norm(x) * (offset + w_next).
    With ``n_parts`` > 1, ``a`` is float32 [n_parts, rows, H] partial sums."""
    n, H = x.shape
    if not (x.is_contiguous() and a.is_contiguous() and (y is None or y.is_contiguous())):
        raise KernelError("add_rmsnorm: tensors must be contiguous")
    part_stride = n * H
    _check(_lib().af_add_rmsnorm(_ptr(x, "x", torch.float32), _ptr(a, "a"), c_int(dtype_code(a.dtype)),
                                 c_int(n_parts), c_longlong(part_stride), _ptr(w_post, "w_post", torch.float32),
                                 _ptr(y, "y", allow_none=True), c_int(dtype_code(y.dtype) if y is not None else F32),
                                 _ptr(w_next, "w_next", torch.float32, allow_none=True),
                                 c_int(n), c_int(H), c_float(eps_post), c_float(eps_next), c_float(offset),
                                 _stream()))


def gated_act(out, gu, activation: str) -> None:
    """out[m, i] = act(gu[m, i]) * gu[m, I + i]."""
    n, inter = out.shape
    if gu.shape != (n, 2 * inter) or not (gu.is_contiguous() and out.is_contiguous()) or gu.dtype != out.dtype:
        raise KernelError("gated_act: gu must be contiguous [rows, 2 * inter] of out's dtype")
    if activation not in ACTIVATIONS:
        raise KernelError(f"gated_act: unknown activation '{activation}' (known: {sorted(ACTIVATIONS)})")
    _check(_lib().af_gated_act(_ptr(out), _ptr(gu), c_int(dtype_code(out.dtype)), c_int(n), c_int(inter),
                               c_int(ACTIVATIONS[activation]), _stream()))


def softcap_(z, cap: float) -> None:
    if not z.is_contiguous():
        raise KernelError("softcap_: tensor must be contiguous")
    _check(_lib().af_softcap(_ptr(z, "z", torch.float32), c_longlong(z.numel()), c_float(cap), _stream()))


# ---------------------------------------------------------------- matrix product

def gemm_plain(out, x, w, cap: float = 0.0) -> None:
    """out[M, N] = x[M, K] @ w[N, K]^T on the CUDA cores, 32-bit accumulation;
    x and w share a dtype, out is that dtype or float32."""
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N) or x.dtype != w.dtype:
        raise KernelError(f"gemm_plain: shapes {tuple(x.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)}")
    _check(_lib().af_gemm_plain(_ptr(out), c_int(dtype_code(out.dtype)), c_int(_rows(out, "out")),
                                _ptr(x), c_int(_rows(x, "x")), _ptr(w), c_int(_rows(w, "w")),
                                c_int(dtype_code(x.dtype)), c_int(M), c_int(N), c_int(K), c_float(cap),
                                _stream()))


# ---------------------------------------------------------------- attention

ROPE_TABLE_ROWS = 64     # from this many rows on, the rotary kernel for bfloat16 rows takes the step's table


def rope_cache_write(qkv, positions, inv_freq, nq: int, nkv: int, hd: int, rot_dim: int, pairing: str,
                     seq_of_token=None, slots=None, len_after=None, kcache=None, vcache=None,
                     page_table=None, ring_rows: int = 0, parts=None, table=None) -> None:
    """Rotate the q and k heads of the packed rows [q | k | v] in place and,
    when a cache is given, store k and v at each token's row of its page.
    ``parts`` (float32 [S, T, width] split-K partial sums) are added into qkv first.
    ``table``: the step's cosines and sines (:func:`rope_table` of these positions and
    frequencies); the kernel for many bfloat16 rows reads them instead of working them
    out for every layer again (the same 32-bit values)."""
    T = qkv.shape[0]
    if qkv.shape[1] != (nq + 2 * nkv) * hd:
        raise KernelError(f"rope_cache_write: row width {qkv.shape[1]} is not (nq + 2 nkv) * head_dim")
    if pairing not in PAIRINGS:
        raise KernelError(f"rope_cache_write: unknown pairing '{pairing}'")
    if inv_freq.numel() != rot_dim // 2:
        raise KernelError("rope_cache_write: inv_freq must hold rot_dim / 2 values")
    if table is not None and (tuple(table.shape) != (T, rot_dim // 2, 2) or not table.is_contiguous()):
        raise KernelError(f"rope_cache_write: the table must be [{T}, {rot_dim // 2}, 2]")
    max_pages = 0
    if kcache is not None:
        if kcache.dtype != qkv.dtype or vcache.dtype != qkv.dtype:
            raise KernelError("rope_cache_write: cache dtype differs from the activations'")
        if tuple(kcache.shape[1:]) != (nkv, PAGE, hd) or not kcache.is_contiguous() or not vcache.is_contiguous():
            raise KernelError(f"rope_cache_write: cache pages must be [pages, {nkv}, {PAGE}, {hd}]")
        max_pages = page_table.shape[1]
    _check(_lib().af_rope_cache_write(
        _ptr(qkv), c_int(dtype_code(qkv.dtype)), c_int(_rows(qkv, "qkv")),
        _ptr(parts, "parts", torch.float32, allow_none=True), c_int(parts.shape[0] if parts is not None else 0),
        c_longlong(parts.stride(0) if parts is not None else 0), _ptr(positions, "positions", torch.int32),
        _ptr(seq_of_token, "seq_of_token", torch.int32, allow_none=True),
        _ptr(slots, "slots", torch.int32, allow_none=True),
        _ptr(len_after, "len_after", torch.int32, allow_none=True),
        _ptr(inv_freq, "inv_freq", torch.float32), _ptr(table, "table", torch.float32, allow_none=True),
        c_int(T), c_int(nq), c_int(nkv), c_int(hd), c_int(rot_dim),
        c_int(PAIRINGS[pairing]), _ptr(kcache, allow_none=True), _ptr(vcache, allow_none=True),
        _ptr(page_table, "page_table", torch.int32, allow_none=True), c_int(max_pages), c_int(ring_rows),
        _stream()))


_EMPTY_F32 = {}


def _no_frequencies(device):
    key = str(device)
    if key not in _EMPTY_F32:
        _EMPTY_F32[key] = torch.empty(0, dtype=torch.float32, device=device)
    return _EMPTY_F32[key]


def no_frequencies(device):
    """An empty table of rotary frequencies (a rotation of no elements)."""
    return _no_frequencies(device)


def store_kv(qkv, batch, nq: int, nkv: int, hd: int, kv, parts=None) -> None:
    """A mixer's cache store: the k and v heads of the packed rows [q | k | v]
    go to each token's row of its cache page (``kv``: the layer's view of its
    pages).  ``parts`` (split-K partial sums of the rows) are added into
    ``qkv`` first.  Nothing is rotated."""
    rope_cache_write(qkv, batch.positions, _no_frequencies(qkv.device), nq, nkv, hd, 0, "half",
                     seq_of_token=batch.seq_of_token, slots=batch.slots, len_after=batch.len_after,
                     kcache=kv.k, vcache=kv.v, page_table=kv.page_table, ring_rows=kv.ring_rows, parts=parts)


def sum_parts(qkv, parts, batch, nq: int, nkv: int, hd: int) -> None:
    """qkv = the sum of the split-K partial sums ``parts`` (float32 [S, T, width]), in index order."""
    rope_cache_write(qkv, batch.positions, _no_frequencies(qkv.device), nq, nkv, hd, 0, "half", parts=parts)


def _gate_args(gate, rows: int, nq: int, who: str):
    """Pointer and row stride of per-head gate logits (float32, row t and head h at [t, h]; columns may be
    a slice of wider rows)."""
    if gate is None:
        return c_void_p(0), c_longlong(0)
    if gate.dtype != torch.float32 or gate.dim() != 2 or gate.shape[0] != rows or gate.shape[1] != nq or gate.stride(1) != 1:
        raise KernelError(f"{who}: gate logits must be float32 [{rows}, {nq}] with unit column stride")
    return _ptr(gate, "gate", torch.float32), c_longlong(gate.stride(0))


def attn_prefill_plain(out, q, k, v, positions, nq: int, nkv: int, hd: int, scale: float, cap: float,
                       window: int, slopes=None, dv=None, mask: str = "window", sinks=None, gate=None) -> None:
    """Attention of prompts that start at position 0 over the step's own keys.
    q [T, nq*hd], k [T, nkv*hd], v [T, nkv*dv] are row views (any row stride; ``dv`` = hd by default).
    ``window`` > 0 with ``mask`` "window": a position sees the last ``window`` ones; "chunk": those of its
    own chunk of ``window`` positions.  ``slopes`` (float32 [nq]): slope[h] * (key position - query position)
    is added to head h's scores after scale and cap (a position encoding that biases scores).  ``sinks``
    (float32 [nq]): exp(sink[h]) joins head h's softmax denominator without a key or a value.  ``gate``
    (float32 [T, nq] logits): head h's output is multiplied by their sigmoid."""
    if slopes is not None and slopes.numel() != nq:
        raise KernelError(f"attn_prefill_plain: {slopes.numel()} slopes for {nq} heads")
    if sinks is not None and sinks.numel() != nq:
        raise KernelError(f"attn_prefill_plain: {sinks.numel()} sinks for {nq} heads")
    if mask not in MASKS:
        raise KernelError(f"attn_prefill_plain: unknown mask '{mask}'")
    T = q.shape[0]
    gp, gs = _gate_args(gate, T, nq, "attn_prefill_plain")
    _check(_lib().af_attn_prefill_plain(
        _ptr(out), c_int(_rows(out, "out")), _ptr(q), c_int(_rows(q, "q")), _ptr(k), c_int(_rows(k, "k")),
        _ptr(v), c_int(_rows(v, "v")), c_int(dtype_code(q.dtype)), _ptr(positions, "positions", torch.int32),
        c_int(T), c_int(nq), c_int(nkv), c_int(hd), c_int(dv or hd), c_float(scale), c_float(cap), c_int(window),
        c_int(MASKS[mask]), _ptr(slopes, "slopes", torch.float32, allow_none=True),
        _ptr(sinks, "sinks", torch.float32, allow_none=True), gp, gs, _stream()))


def plain_decode_splits(batch: int, nq: int, most_keys: int) -> int:
    """Into how many runs the plain decode kernel cuts a sequence's visible keys (a warp a run): enough warps
    for the device's SMs to have some thirty each, no run shorter than 32 keys."""
    want = -(-sm_count() * 32 // max(1, batch * nq))
    return max(1, min(want, most_keys // 32, 256))


def attn_decode_plain(out, q, kcache, vcache, page_table, slots, lens, nq: int, nkv: int, hd: int,
                      scale: float, cap: float, window: int, ring_rows: int, slopes=None, dv=None,
                      mask: str = "window", sinks=None, gate=None, n_splits: int = 1) -> None:
    """Attention of one new token per sequence over the cache pages (options as in
    :func:`attn_prefill_plain`).  ``vcache`` None: a value is the first ``dv`` elements of its key row.
    ``n_splits`` > 1: a sequence's visible keys are cut into that many runs, a warp each, joined by a
    second kernel."""
    B = q.shape[0]
    if slopes is not None and slopes.numel() != nq:
        raise KernelError(f"attn_decode_plain: {slopes.numel()} slopes for {nq} heads")
    if sinks is not None and sinks.numel() != nq:
        raise KernelError(f"attn_decode_plain: {sinks.numel()} sinks for {nq} heads")
    if mask not in MASKS:
        raise KernelError(f"attn_decode_plain: unknown mask '{mask}'")
    if kcache.dtype != q.dtype:
        raise KernelError("attn_decode_plain: cache dtype differs from the activations'")
    dv = dv or hd
    if tuple(kcache.shape[1:]) != (nkv, PAGE, hd) or (vcache is not None and tuple(vcache.shape[1:]) != (nkv, PAGE, dv)):
        raise KernelError(f"attn_decode_plain: cache pages must be [pages, {nkv}, {PAGE}, {hd}] (values {dv})")
    gp, gs = _gate_args(gate, B, nq, "attn_decode_plain")
    scratch = torch.empty(B * nq * n_splits * (dv + 2), dtype=torch.float32, device=q.device) if n_splits > 1 else None
    _check(_lib().af_attn_decode_plain(
        _ptr(out), c_int(_rows(out, "out")), _ptr(q), c_int(_rows(q, "q")), _ptr(kcache),
        _ptr(vcache, allow_none=True),
        c_int(dtype_code(q.dtype)), _ptr(page_table, "page_table", torch.int32), c_int(page_table.shape[1]),
        _ptr(slots, "slots", torch.int32), _ptr(lens, "lens", torch.int32), c_int(B), c_int(nq), c_int(nkv),
        c_int(hd), c_int(dv), c_float(scale), c_float(cap), c_int(window), c_int(MASKS[mask]), c_int(ring_rows),
        _ptr(slopes, "slopes", torch.float32, allow_none=True), _ptr(sinks, "sinks", torch.float32, allow_none=True),
        gp, gs, c_int(n_splits), _ptr(scratch, "scratch", torch.float32, allow_none=True), _stream()))


def add_(x, a) -> None:
    """x += a; x float32, a float32 or bfloat16, same shape (or [S, *x.shape]
    partial sums, added one after the other)."""
    if a.dim() == x.dim() + 1:
        for part in a:
            add_(x, part)
        return
    if x.shape != a.shape or not (x.is_contiguous() and a.is_contiguous()):
        raise KernelError("add_: tensors must be contiguous and of one shape")
    _check(_lib().af_add(_ptr(x, "x", torch.float32), _ptr(a), c_int(dtype_code(a.dtype)),
                         c_longlong(x.numel()), _stream()))


def sample(logits, out, temperature: float, top_p: float, penalty: float, uniform=None, recent=None,
           n_recent=None) -> None:
    """One token per row of float32 logits [R, V] into out int32 [R].  The
    repetition penalty changes ``logits`` in place.  ``recent`` int32 [R, 64]
    holds each row's last tokens, ``n_recent`` int32 [R] how many are valid,
    ``uniform`` float32 [R] the draws in [0, 1)."""
    R, V = logits.shape
    if out.shape[0] != R:
        raise KernelError("sample: one output per row")
    _check(_lib().af_sample(_ptr(logits, "logits", torch.float32), c_int(_rows(logits, "logits")), c_int(R),
                            c_int(V), _ptr(recent, "recent", torch.int32, allow_none=True),
                            _ptr(n_recent, "n_recent", torch.int32, allow_none=True),
                            c_int(recent.stride(0) if recent is not None else 0), c_float(temperature),
                            c_float(top_p), c_float(penalty),
                            _ptr(uniform, "uniform", torch.float32, allow_none=True),
                            _ptr(out, "out", torch.int32), _stream()))


_ERR = {}


def error_word(device) -> torch.Tensor:
    """The device word that kernels set when a bounded wait inside them ran out."""
    key = torch.device(device).index or 0
    if key not in _ERR:
        _ERR[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _ERR[key]


def check_device_errors(device) -> None:
    """Raise if a kernel reported a wait that ran out of time (reads one word: synchronises)."""
    w = error_word(device)
    if int(w.item()) != 0:
        w.zero_()
        raise KernelError("a tensor-core kernel gave up waiting on a barrier (results of the step are invalid)")


def selftest_wait_runs_out(device, limit_ms: float = 2.0) -> float:
    """Runs a kernel whose wait on a barrier nobody arrives on gives up after
    ``limit_ms`` and sets the device's error word, as the tensor-core kernels'
    waits do after their limit.  Returns the milliseconds the wait took; the
    error word is left set (``check_device_errors`` raises and clears it)."""
    waited = torch.zeros(1, dtype=torch.int64, device=device)
    _check(_lib().af_selftest_wait_runs_out(_ptr(error_word(device), "err", torch.int32),
                                            ctypes.c_ulonglong(int(limit_ms * 1e6)), _ptr(waited), _stream()))
    return float(waited.item()) / 1e6


def gemm_tc_supported(x, w, out) -> bool:
    """Whether the tensor-core product takes these operands: bfloat16, dense
    rows, K and row strides multiples of 8, 16-byte aligned bases."""
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        return False
    if x.dim() != 2 or w.dim() != 2 or x.stride(1) != 1 or w.stride(1) != 1:
        return False
    K = x.shape[1]
    return (K % 8 == 0 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0
            and w.data_ptr() % 16 == 0 and (out is None or out.stride(-1) == 1))


def gemm_tc_splits(M: int, N: int, K: int) -> int:
    """How many K splits fill the GPU when a product has few output tiles: up to
    two blocks an SM (a grid beyond one wave runs two blocks an SM, which stream
    at once: measured faster inside the decode step than one wave of blocks
    with a whole SM each; for up to 16 rows), at least 4 K blocks a split, at
    most 16 splits."""
    lib = _lib()
    bn = lib.af_gemm_tc_token_tile(c_int(M))
    tiles = ((N + 127) // 128) * ((M + bn - 1) // bn)
    kb = (K + 63) // 64
    if tiles >= 96 or kb < 8:
        return 1
    waves = 2 if M <= 16 else 1       # (more rows: the partial sums' own bytes weigh more than the fuller GPU)
    want = max(1, min((waves * sm_count()) // tiles, kb // 4, 16))
    per = (kb + want - 1) // want
    return (kb + per - 1) // per


# Blocks per SM of the weight-bound product (up to 64 tokens): 0 lets the library choose.
GEMM_TC_PER_SM = 0


def gemm_tc(out, x, w, cap: float = 0.0, splits: int = 1, gated: bool = False, activation: str = "gelu_tanh",
            n_acc: int = 0, checked: bool = False, per_sm: int = -1) -> None:
    """out = x @ w^T on the tcgen05 tensor cores (bfloat16 operands, 32-bit
    accumulation in TMEM).  splits > 1: out is float32 [splits, M, N] partial
    sums.  gated: w holds, per group of 32 rows, 16 gate rows then the 16 up
    rows of the same features (see ``interleave_gate_up``); out[m, f] =
    act(x . gate_f) * (x . up_f), N = rows / 2.  n_acc: weight tiles per block
    (1 or 2), or 4: the kernel that runs a tile on a pair of SMs
    (``tcgen05.mma.cta_group::2``, two accumulators in turn: for prompts);
    0: chosen from the sizes.  ``checked``: the caller has asked
    :func:`gemm_tc_supported` already."""
    M, K = x.shape
    rows = w.shape[0]
    N = rows // 2 if gated else rows
    if not checked and not gemm_tc_supported(x, w, out):
        raise KernelError("gemm_tc: operands must be bfloat16 with dense, 16-byte aligned rows and K % 8 == 0")
    if splits > 1:
        if out.dtype != torch.float32 or tuple(out.shape) != (splits, M, N) or not out.is_contiguous():
            raise KernelError("gemm_tc: split-K wants a contiguous float32 [splits, M, N] output")
        ldo, part = N, M * N
    else:
        if tuple(out.shape) != (M, N):
            raise KernelError(f"gemm_tc: output shape {tuple(out.shape)}, expected {(M, N)}")
        ldo, part = out.stride(0), 0
    if n_acc == 0:
        # Many tokens.  Two weight tiles per block halve the bytes a block stages per flop; worth it once the
        # tiles of 256 x 256 fill the GPU.  With fewer tiles and a long K a tile runs on a pair of SMs (the same
        # bytes per flop, 128 rows a block); with a short K the pair's set-up costs what it saves.  Measured at
        # 2,048 tokens on a B200: 18432 x 2304 gated 122 us / 124 us / 132 us (two tiles / pair / one tile),
        # 2304 x 9216 90 / 59 / 63, 2304 x 2048 25 / 17 / 15, 4096 x 2304 31 / 31 / 31.
        blocks2 = ((rows + 255) // 256) * ((M + 255) // 256)
        n_acc = 1
        if M > 128 and splits == 1:
            if blocks2 >= 120:
                n_acc = 2
            elif blocks2 >= 60 and K >= 4096:
                n_acc = 4
    if n_acc == 4:
        if splits > 1:
            raise KernelError("gemm_tc: the kernel on pairs of SMs does not split K")
        _check(_lib().af_gemm_tc_pair(_ptr(out), c_int(dtype_code(out.dtype)), c_longlong(ldo), _ptr(x),
                                      c_longlong(x.stride(0)), _ptr(w), c_longlong(w.stride(0)), c_longlong(rows),
                                      c_int(M), c_int(K), c_int(1 if gated else 0), c_int(ACTIVATIONS[activation]),
                                      c_float(cap), _ptr(error_word(x.device), "err", torch.int32), _stream()))
        return
    _check(_lib().af_gemm_tc(_ptr(out), c_int(dtype_code(out.dtype)), c_longlong(ldo), c_longlong(part), _ptr(x),
                             c_longlong(x.stride(0)), _ptr(w), c_longlong(w.stride(0)), c_longlong(rows),
                             c_int(M), c_int(K), c_int(1 if gated else 0), c_int(ACTIVATIONS[activation]),
                             c_int(n_acc), c_float(cap), c_int(splits), c_int(GEMM_TC_PER_SM if per_sm < 0 else per_sm),
                             _ptr(error_word(x.device), "err", torch.int32), _stream()))


def rope_table(positions, inv_freq) -> torch.Tensor:
    """float32 [T, pairs, 2]: (cos, sin) of position * frequency for every token
    of the step and every rotary pair (32-bit angles)."""
    T, half = positions.shape[0], inv_freq.numel()
    table = torch.empty(T, half, 2, dtype=torch.float32, device=positions.device)
    _check(_lib().af_rope_table(_ptr(table), _ptr(positions, "positions", torch.int32),
                                _ptr(inv_freq, "inv_freq", torch.float32), c_int(T), c_int(half), _stream()))
    return table


def rope_table_precise(positions, inv_freq64) -> torch.Tensor:
    """The same table from float64 frequencies with the angle and its reduction in 64 bits."""
    T, half = positions.shape[0], inv_freq64.numel()
    table = torch.empty(T, half, 2, dtype=torch.float32, device=positions.device)
    _check(_lib().af_rope_table_precise(_ptr(table), _ptr(positions, "positions", torch.int32),
                                        _ptr(inv_freq64, "inv_freq", torch.float64), c_int(T), c_int(half), _stream()))
    return table


def kv_rows(batch, kv, nkv: int) -> torch.Tensor:
    """int32 [T]: each token's row in the cache pages of ``kv`` (a layer's view;
    all layers of its group share the page table) for kv head 0, -1 for tokens
    that are not stored."""
    T = batch.tokens.shape[0]
    rows = torch.empty(T, dtype=torch.int32, device=batch.tokens.device)
    _check(_lib().af_kv_rows(_ptr(rows), _ptr(batch.positions, "positions", torch.int32),
                             _ptr(batch.seq_of_token, "seq_of_token", torch.int32),
                             _ptr(batch.slots, "slots", torch.int32), _ptr(batch.len_after, "len_after", torch.int32),
                             _ptr(kv.page_table, "page_table", torch.int32), c_int(kv.page_table.shape[1]),
                             c_int(kv.ring_rows), c_int(nkv), c_int(T), _stream()))
    return rows


def rope_row_order(n_heads: int, hd: int, device=None) -> torch.Tensor:
    """The order of a packed [q | k | v] weight's rows that :func:`gemm_tc_rope`
    wants: within every head, groups of 32 rows, each the 16 rows p .. p + 15
    of the head's first half followed by the rows p + hd / 2 .. that they are
    rotated with.  Returns the old row index of every new row (int64)."""
    if hd % 32:
        raise KernelError(f"rope_row_order: head_dim {hd} is not a multiple of 32")
    i = torch.arange(hd, device=device)
    within = (i // 32) * 16 + i % 16 + (i % 32 >= 16) * (hd // 2)
    return (torch.arange(n_heads, device=device)[:, None] * hd + within[None, :]).reshape(-1)


def gemm_tc_rope_supported(x, w, hd: int) -> bool:
    return hd % 32 == 0 and gemm_tc_supported(x, w, None)


def gemm_tc_rope(out, x, w, table, nq: int, nkv: int, hd: int, rows=None, kcache=None, vcache=None,
                 splits: int = 1, tickets=None, n_acc: int = 0, per_sm: int = -1) -> None:
    """out [M, (nq + 2 nkv) hd] bfloat16 = x @ w^T with the rotary encoding and
    the cache write in the product's epilogue: ``w`` holds the rows in
    :func:`rope_row_order`, ``table`` is :func:`rope_table` of the step; q and k
    heads are rotated (pairs i, i + hd / 2), v is not; ``out`` is in the plain
    order.  With ``rows`` (:func:`kv_rows`) and the layer's cache pages, k and v
    also go to each token's cache row.  ``splits`` > 1 (up to 64 tokens): the
    last block of a tile to finish adds the partial tiles in index order;
    ``tickets`` is a zeroed int32 tensor that the kernel leaves zeroed."""
    M, K = x.shape
    N = w.shape[0]
    if out.dtype != torch.bfloat16 or tuple(out.shape) != (M, N) or N != (nq + 2 * nkv) * hd:
        raise KernelError(f"gemm_tc_rope: output {tuple(out.shape)} for {(M, (nq + 2 * nkv) * hd)}")
    if not gemm_tc_rope_supported(x, w, hd):
        raise KernelError("gemm_tc_rope: operands must be bfloat16 with dense, 16-byte aligned rows, K % 8 == 0 "
                          "and head_dim % 32 == 0")
    if tuple(table.shape) != (M, hd // 2, 2) or table.dtype != torch.float32 or not table.is_contiguous():
        raise KernelError(f"gemm_tc_rope: the table must be float32 [{M}, {hd // 2}, 2]")
    if rows is not None:
        if kcache is None or vcache is None or kcache.dtype != torch.bfloat16 or not kcache.is_contiguous() \
                or tuple(kcache.shape[1:]) != (nkv, PAGE, hd) or vcache.shape != kcache.shape:
            raise KernelError(f"gemm_tc_rope: cache pages must be bfloat16 [pages, {nkv}, {PAGE}, {hd}]")
    parts = None
    if splits > 1:
        need = int(_lib().af_gemm_tc_rope_tickets(c_int(M), c_longlong(N)))
        if M > 64 or tickets is None or tickets.dtype != torch.int32 or tickets.numel() < need:
            raise KernelError(f"gemm_tc_rope: split-K serves up to 64 tokens and needs {need} zeroed int32 tickets")
        parts = torch.empty(splits, M, N, dtype=torch.float32, device=x.device)
    if n_acc == 0:
        blocks2 = ((N + 255) // 256) * ((M + 255) // 256)
        n_acc = 2 if (M > 128 and splits == 1 and blocks2 >= 120) else 1
    _check(_lib().af_gemm_tc_rope(
        _ptr(out), c_longlong(out.stride(0)), _ptr(x), c_longlong(x.stride(0)), _ptr(w), c_longlong(w.stride(0)),
        c_longlong(N), c_int(M), c_int(K), c_int(n_acc), c_int(splits),
        _ptr(parts, "parts", torch.float32, allow_none=True), _ptr(tickets, "tickets", torch.int32, allow_none=True),
        _ptr(table, "table", torch.float32), _ptr(rows, "rows", torch.int32, allow_none=True),
        _ptr(kcache, allow_none=True), _ptr(vcache, allow_none=True), c_int(hd), c_int(nq), c_int(nkv),
        c_int(GEMM_TC_PER_SM if per_sm < 0 else per_sm), _ptr(error_word(x.device), "err", torch.int32), _stream()))


def argmax_key_stride() -> int:
    """64-bit words between the keys of two rows of :func:`gemm_tc_argmax`."""
    return int(_lib().af_argmax_key_stride())


def gemm_tc_argmax(tokens, x, w, cap: float, keys) -> None:
    """tokens[m] = argmax over the rows n of softcap(x[m] . w[n]) (finite values
    only, the lowest row among equals, 0 when none is finite), without the
    logits going to memory: the product's epilogue joins every block's best
    into one 64-bit key per token.  ``keys``: int64 [>= M] on the device, zero
    before the call and zero again after it."""
    M, K = x.shape
    if not gemm_tc_supported(x, w, None):
        raise KernelError("gemm_tc_argmax: operands must be bfloat16 with dense, 16-byte aligned rows and K % 8 == 0")
    if tokens.dtype != torch.int32 or tokens.numel() < M or keys.dtype != torch.int64 \
            or keys.numel() < M * argmax_key_stride():
        raise KernelError("gemm_tc_argmax: int32 tokens, one per row, and int64 keys, argmax_key_stride() per row")
    lib = _lib()
    _check(lib.af_gemm_tc_argmax(_ptr(keys), _ptr(x), c_longlong(x.stride(0)), _ptr(w), c_longlong(w.stride(0)),
                                 c_longlong(w.shape[0]), c_int(M), c_int(K), c_float(cap), c_int(max(GEMM_TC_PER_SM, 0)),
                                 _ptr(error_word(x.device), "err", torch.int32), _stream()))
    _check(lib.af_argmax_finish(_ptr(tokens), _ptr(keys), c_int(M), _stream()))


def interleave_gate_up(w_gate, w_up):
    """The gated product's weight layout: groups of 32 rows, each 16 gate rows
    followed by the up rows of the same 16 features.  Rows beyond the last
    whole 16 are padded with zeros (their outputs are never written)."""
    inter, K = w_gate.shape
    groups = (inter + 15) // 16
    out = torch.zeros(groups * 32, K, dtype=w_gate.dtype, device=w_gate.device)
    v = out.view(groups, 2, 16, K)
    pad = groups * 16 - inter
    if pad:
        g = torch.cat([w_gate, torch.zeros(pad, K, dtype=w_gate.dtype, device=w_gate.device)])
        u = torch.cat([w_up, torch.zeros(pad, K, dtype=w_up.dtype, device=w_up.device)])
    else:
        g, u = w_gate, w_up
    v[:, 0] = g.view(groups, 16, K)
    v[:, 1] = u.view(groups, 16, K)
    return out

def attn_prefill_mma(out, q, k, v, seq_starts, n_seqs: int, max_len: int, nq, nkv, hd, scale, cap, window,
                     sinks=None, gate=None) -> None:
    """bfloat16 prefill attention on the tensor cores; sequences packed row
    after row, ``seq_starts`` int32 [n_seqs + 1].  ``sinks`` and ``gate`` as in :func:`attn_prefill_plain`."""
    gp, gs = _gate_args(gate, q.shape[0], nq, "attn_prefill_mma")
    if q.dtype != torch.bfloat16 or k.dtype != torch.bfloat16 or v.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("attn_prefill_mma: bfloat16 only")
    _check(_lib().af_attn_prefill(
        _ptr(out), c_longlong(_rows(out, "out")), _ptr(q), c_longlong(_rows(q, "q")), _ptr(k),
        c_longlong(_rows(k, "k")), _ptr(v), c_longlong(_rows(v, "v")), _ptr(seq_starts, "seq_starts", torch.int32),
        c_int(n_seqs), c_int(max_len), c_int(nq), c_int(nkv), c_int(hd), c_float(scale), c_float(cap), c_int(window),
        _ptr(sinks, "sinks", torch.float32, allow_none=True), gp, gs, _stream()))


def attn_prefill_tc(out, q, k, v, seq_starts, n_seqs: int, max_len: int, nq, nkv, hd, scale, cap, window,
                    sinks=None, gate=None) -> None:
    """bfloat16 prefill attention on tcgen05 (S and O in TMEM); sequences packed
    row after row, ``seq_starts`` int32 [n_seqs + 1].  ``sinks`` and ``gate`` as in :func:`attn_prefill_plain`."""
    gp, gs = _gate_args(gate, q.shape[0], nq, "attn_prefill_tc")
    if q.dtype != torch.bfloat16 or k.dtype != torch.bfloat16 or v.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("attn_prefill_tc: bfloat16 only")
    if k.shape[0] != q.shape[0] or v.shape[0] != q.shape[0]:
        raise KernelError("attn_prefill_tc: q, k and v hold the same rows")
    _check(_lib().af_attn_prefill_tc(
        _ptr(out), c_longlong(_rows(out, "out")), _ptr(q), c_longlong(_rows(q, "q")), _ptr(k),
        c_longlong(_rows(k, "k")), _ptr(v), c_longlong(_rows(v, "v")), _ptr(seq_starts, "seq_starts", torch.int32),
        c_int(n_seqs), c_int(q.shape[0]), c_int(max_len), c_int(nq), c_int(nkv), c_int(hd), c_float(scale),
        c_float(cap), c_int(window), _ptr(sinks, "sinks", torch.float32, allow_none=True), gp, gs,
        _ptr(error_word(q.device), "err", torch.int32), _stream()))


def head_gate(x, gate, nq: int, dv: int) -> None:
    """x[t, h, :] *= sigmoid(gate[t, h]) for rows x [T, nq dv] (an output gate behind an attention kernel that
    has none of its own)."""
    T = x.shape[0]
    gp, gs = _gate_args(gate, T, nq, "head_gate")
    _check(_lib().af_head_gate(_ptr(x), c_longlong(_rows(x, "x")), c_int(dtype_code(x.dtype)), gp, gs, c_int(T),
                               c_int(nq), c_int(dv), _stream()))


def _chunk_starts(batch, size: int):
    """The rows at which the chunks of ``size`` positions of a prefill step's sequences begin (int32 on the
    device, one more than there are chunks), how many chunks there are and the longest: under a chunked mask every
    chunk is a causal sequence of its own.  Made once a step (kept in ``batch.aux``)."""
    key = ("chunk_starts", size)
    if key not in batch.aux:
        starts, row = [], 0
        for n in batch.seq_lens:
            starts.extend(range(row, row + n, size))
            row += n
        starts.append(row)
        host = torch.tensor(starts, dtype=torch.int32)
        batch.aux[key] = (host.to(batch.tokens.device), len(starts) - 1, min(size, max(batch.seq_lens)))
    return batch.aux[key]


def attn_prefill(out, q, k, v, batch, nq, nkv, hd, scale, cap, window, slopes=None, dv=None, mask: str = "window",
                 sinks=None, gate=None) -> None:
    """Attention of a prefill step: for bfloat16 the tcgen05 kernel (head sizes
    128, 256) or the mma.sync kernel (64), else the plain kernel (which also
    serves scores with a per-head slope and values of another size than the keys).  A chunked mask
    reaches the fast kernels as what it is: causal attention within chunks that know nothing of one another."""
    fast = q.dtype == torch.bfloat16 and slopes is None and (dv or hd) == hd
    aligned = all(t.stride(0) % 8 == 0 and t.data_ptr() % 16 == 0 for t in (q, k, v, out))
    use_tc = fast and aligned and bool(_lib().af_attn_prefill_tc_supported(c_int(hd)))
    use_mma = fast and not use_tc and bool(_lib().af_attn_prefill_supported(c_int(hd))) \
        and all(t.stride(0) % 8 == 0 and t.data_ptr() % 16 == 0 for t in (q, k, v))
    if not (use_tc or use_mma):
        attn_prefill_plain(out, q, k, v, batch.positions, nq, nkv, hd, scale, cap, window, slopes, dv=dv, mask=mask,
                           sinks=sinks, gate=gate)
        return
    starts, n_seqs, max_len, size = batch.seq_starts, batch.n_seqs, batch.max_len, window
    if mask == "chunk" and window:
        starts, n_seqs, max_len = _chunk_starts(batch, window)
        window = 0
    if n_seqs > 65535:          # (more sequences than a grid's second axis takes)
        attn_prefill_plain(out, q, k, v, batch.positions, nq, nkv, hd, scale, cap, size, slopes, dv=dv, mask=mask,
                           sinks=sinks, gate=gate)
    elif use_tc:
        attn_prefill_tc(out, q, k, v, starts, n_seqs, max_len, nq, nkv, hd, scale, cap, window, sinks, gate)
    else:
        attn_prefill_mma(out, q, k, v, starts, n_seqs, max_len, nq, nkv, hd, scale, cap, window, sinks, gate)


def attn_decode_max_splits(batch: int, nkv: int, max_len: int, window: int, blocks: int = 0, nq: int = 0) -> int:
    """The most splits the decode kernel may give one (sequence, kv head) unit:
    the room its partial results need.  The kernel's blocks (one an SM) each
    take an equal share of all units' cache pages, so a unit lies in at most
    ``blocks // units of a sequence + 2`` blocks (one long sequence among empty
    ones, whatever the batch) and in at most its pages + 1."""
    blocks = blocks or sm_count()
    window = abs(window)            # (negative: a chunk of that many positions)
    rows = min(max_len, window) if window else max_len
    pages = max(1, (rows + PAGE - 1) // PAGE + (1 if window else 0))
    tiles = ((nq // nkv) + 15) // 16 if nq else 1
    return max(1, min(blocks // max(1, nkv * tiles) + 2, pages + 1))


def attn_decode_plan(page_table, slots, lens, nq: int, nkv: int, window: int, ring_rows: int, n_splits: int):
    """The plan of a decode step for :func:`attn_decode_split`: how the work is
    cut among the blocks, worked out by one small kernel for all layers that
    read the same caches the same way (these slots, lengths, page table, heads,
    window, ring and ``n_splits``).  It holds for these lengths alone."""
    lib = _lib()
    lib.af_attn_decode_plan_ints.restype = ctypes.c_longlong
    B = slots.shape[0]
    n = lib.af_attn_decode_plan_ints(c_int(B), c_int(nq), c_int(nkv))
    if n <= 0:
        raise KernelError(f"attn_decode_plan: {B} sequences, {nq} heads in {nkv} groups")
    plan = torch.empty(n, dtype=torch.int32, device=slots.device)
    _check(lib.af_attn_decode_plan(
        _ptr(plan, "plan", torch.int32), c_longlong(n), _ptr(page_table, "page_table", torch.int32),
        c_int(page_table.shape[1]), _ptr(slots, "slots", torch.int32), _ptr(lens, "lens", torch.int32), c_int(B),
        c_int(nq), c_int(nkv), c_int(window), c_int(ring_rows), c_int(n_splits), _stream()))
    return plan


def attn_decode_split(out, q, kcache, vcache, page_table, slots, lens, nq, nkv, hd, scale, cap, window, ring_rows,
                      n_splits: int, scratch=None, plan=None, sinks=None) -> None:
    """bfloat16 decode attention, split over the keys (two kernels: partial
    results into ``scratch``, then their merge).  ``n_splits`` is the most
    splits a (sequence, kv head) unit gets: the kernel cuts the units' pages so
    that all blocks get about the same number of them (with less room than
    :func:`attn_decode_max_splits` fewer blocks work)."""
    B = q.shape[0]
    lib = _lib()
    lib.af_attn_decode_scratch.restype = ctypes.c_longlong
    need = lib.af_attn_decode_scratch(c_int(B), c_int(nq), c_int(hd), c_int(n_splits))
    if scratch is None:
        scratch = torch.empty(need, dtype=torch.float32, device=q.device)
    elif scratch.numel() < need or scratch.dtype != torch.float32:
        raise KernelError(f"attn_decode_split: scratch of {need} floats wanted")
    if q.dtype != torch.bfloat16 or kcache.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("attn_decode_split: bfloat16 only")
    if sinks is not None and sinks.numel() != nq:
        raise KernelError(f"attn_decode_split: {sinks.numel()} sinks for {nq} heads")
    _check(lib.af_attn_decode_sinks(
        _ptr(out), c_longlong(_rows(out, "out")), _ptr(q), c_longlong(_rows(q, "q")), _ptr(kcache), _ptr(vcache),
        c_longlong(kcache.shape[0]), _ptr(page_table, "page_table", torch.int32), c_int(page_table.shape[1]),
        _ptr(slots, "slots", torch.int32),
        _ptr(lens, "lens", torch.int32), c_int(B), c_int(nq), c_int(nkv), c_int(hd), c_float(scale), c_float(cap),
        c_int(window), c_int(ring_rows), c_int(n_splits), _ptr(scratch, "scratch", torch.float32),
        _ptr(plan, "plan", torch.int32) if plan is not None else ctypes.c_void_p(0),
        _ptr(sinks, "sinks", torch.float32, allow_none=True),
        _ptr(error_word(q.device), "err", torch.int32), _stream()))


def attn_decode_latent_supported(dtype, hd: int, dv: int) -> bool:
    """Whether :func:`attn_decode_latent` takes cached rows of ``hd`` elements with the values their first ``dv``."""
    return dtype == torch.bfloat16 and bool(_lib().af_attn_decode_latent_supported(c_int(hd), c_int(dv)))


def attn_decode_latent(out, q, kcache, page_table, slots, lens, nq: int, nkv: int, hd: int, dv: int, scale: float,
                       window: int, ring_rows: int, mask: str = "window", sinks=None, gate=None, n_splits: int = 1) -> None:
    """bfloat16 decode attention over cached rows that hold their values inside their keys (a value: the first
    ``dv`` elements of its key row of ``hd``), on the tensor cores, the query heads of a kv head sharing every row
    read; the visible keys cut into ``n_splits`` runs, joined by the plain kernel's merge (sinks and gate there)."""
    B = q.shape[0]
    if q.dtype != torch.bfloat16 or kcache.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("attn_decode_latent: bfloat16 only")
    if tuple(kcache.shape[1:]) != (nkv, PAGE, hd) or not kcache.is_contiguous() or tuple(out.shape) != (B, nq * dv):
        raise KernelError(f"attn_decode_latent: cache pages [pages, {nkv}, {PAGE}, {hd}], out [{B}, {nq * dv}]")
    if mask not in MASKS or (sinks is not None and sinks.numel() != nq):
        raise KernelError("attn_decode_latent: mask, or one sink a head")
    gp, gs = _gate_args(gate, B, nq, "attn_decode_latent")
    scratch = torch.empty(B * nq * n_splits * (dv + 2), dtype=torch.float32, device=q.device)
    part_o, part_ml = scratch[: B * nq * n_splits * dv], scratch[B * nq * n_splits * dv:]
    _check(_lib().af_attn_decode_latent(
        _ptr(q), c_longlong(_rows(q, "q")), _ptr(kcache), _ptr(page_table, "page_table", torch.int32),
        c_int(page_table.shape[1]), _ptr(slots, "slots", torch.int32), _ptr(lens, "lens", torch.int32), c_int(B), c_int(nq),
        c_int(nkv), c_int(hd), c_int(dv), c_float(scale), c_int(window), c_int(MASKS[mask]), c_int(ring_rows),
        c_int(n_splits), _ptr(part_o), _ptr(part_ml), _stream()))
    _check(_lib().af_attn_decode_merge_runs(
        _ptr(out), c_int(_rows(out, "out")), c_int(dtype_code(out.dtype)), _ptr(part_o), _ptr(part_ml),
        _ptr(slots, "slots", torch.int32), c_int(B), c_int(nq), c_int(dv), c_int(n_splits),
        _ptr(sinks, "sinks", torch.float32, allow_none=True), gp, gs, _stream()))


ATTN_DECODE_MAX_SEQS = 2048     # sequences of a step that the split kernel plans for (more: the plain kernel)


def attn_decode_fast(dtype, hd: int, n_seqs: int) -> bool:
    """Whether :func:`attn_decode` has the split kernel for these sizes."""
    return dtype == torch.bfloat16 and bool(_lib().af_attn_decode_supported(c_int(hd))) and n_seqs <= ATTN_DECODE_MAX_SEQS


def attn_decode(out, q, kv, batch, nq, nkv, hd, scale, cap, window, slopes=None, dv=None, mask: str = "window",
                sinks=None, gate=None) -> None:
    """Attention of a decode step over the cache: the split kernel for
    bfloat16 and head sizes it takes (a chunked mask goes to it as a negative window, a gate follows it as a
    kernel of its own), else the plain kernel (which also serves scores with a per-head slope, values of another
    size than the keys or inside them, and sinks)."""
    # values that lie inside their key rows: the split kernel takes the key pages for the value pages too and gives
    # whole key-sized rows back, of which the caller (who asked for it with an `out` that wide) reads the values' part
    wide = kv.v is None and out.shape[1] == nq * hd
    special = slopes is not None or (not wide and ((dv or hd) != hd or kv.v is None))
    if (not special and q.dtype == torch.bfloat16 and _lib().af_attn_decode_supported(c_int(hd))
            and batch.n_seqs <= ATTN_DECODE_MAX_SEQS):
        if mask == "chunk":
            window = -window
        n = attn_decode_max_splits(batch.n_seqs, nkv, batch.max_len_after, window, nq=nq)
        # the plan of the step, shared by the layers that read this group of caches alike (a batch without a
        # place for the step's tables gets none: every block then works the cut out itself)
        plan, aux = None, getattr(batch, "aux", None)
        if aux is not None:
            key = ("attn_decode_plan", kv.page_table.data_ptr(), kv.ring_rows, nq, nkv, window, n)
            if key not in aux:
                aux[key] = attn_decode_plan(kv.page_table, batch.slots, batch.len_after, nq, nkv, window,
                                            kv.ring_rows, n)
            plan = aux[key]
        attn_decode_split(out, q, kv.k, kv.k if wide else kv.v, kv.page_table, batch.slots, batch.len_after, nq, nkv,
                          hd, scale, cap, window, kv.ring_rows, n, plan=plan, sinks=sinks)
        if gate is not None:
            head_gate(out, gate, nq, hd)
        return
    # (a captured step sizes its cut for the longest context; the keys a token sees are bounded by its window or chunk)
    most = min(batch.max_len_after, window) if window else batch.max_len_after
    if (kv.v is None and slopes is None and cap == 0.0 and attn_decode_latent_supported(q.dtype, hd, dv or hd)
            and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0 and batch.n_seqs < 65536):
        # wide rows with the values inside: the tensor-core kernel, runs of at least 64 keys, some two blocks an SM
        units = batch.n_seqs * nkv * ((nq // nkv + 15) // 16)
        n = max(1, min(-(-2 * sm_count() // units), -(-most // 64), 256))
        attn_decode_latent(out, q, kv.k, kv.page_table, batch.slots, batch.len_after, nq, nkv, hd, dv or hd, scale,
                           window, kv.ring_rows, mask=mask, sinks=sinks, gate=gate, n_splits=n)
        return
    attn_decode_plain(out, q, kv.k, kv.v, kv.page_table, batch.slots, batch.len_after, nq, nkv, hd,
                      scale, cap, window, kv.ring_rows, slopes, dv=dv, mask=mask, sinks=sinks, gate=gate,
                      n_splits=plain_decode_splits(batch.n_seqs, nq, most))


# ---------------------------------------------------------------- mixers with a state of fixed size

SCAN_MODES = {"decay": 0, "delta": 1, "channel": 3}


def _f32_rows(t, name):
    """Pointer and token stride of float32 rows (a column section of a packed projection is fine)."""
    if t.dtype != torch.float32 or t.dim() != 2 or t.stride(1) != 1:
        raise KernelError(f"{name} must be float32 rows, got {t.dtype} {tuple(t.shape)} strides {t.stride()}")
    return _ptr(t, name), c_longlong(t.stride(0))


def delta_prep(out, proj, off_k: int, off_a: int, off_w1: int, a_bias, w0, w2t, heads: int, dk: int,
               decay_scale: float, key_eps: float) -> None:
    """What enters the generalized delta rule besides r, k and v, from the packed float32 projection rows
    ``proj`` (sections at the given column offsets): out [T, 3, heads * dk] float32 = the decay
    exp(-decay_scale * sigmoid(w2 tanh(w1 section) + w0)), the unit key k / sqrt(sum k^2 + key_eps) per head,
    and sigmoid(a section + a_bias) times the unit key.  ``w2t`` is w2 transposed: [rank, heads * dk]."""
    T = proj.shape[0]
    n = heads * dk
    rank = w2t.shape[0]
    if tuple(out.shape) != (T, 3, n) or out.dtype != torch.float32 or not out.is_contiguous():
        raise KernelError(f"delta_prep: out must be contiguous float32 [{T}, 3, {n}]")
    if tuple(w2t.shape) != (rank, n) or not w2t.is_contiguous() or a_bias.numel() != n or w0.numel() != n:
        raise KernelError("delta_prep: w2t [rank, heads * dk], a_bias and w0 [heads * dk]")
    if max(off_k, off_a) + n > proj.shape[1] or off_w1 + rank > proj.shape[1]:
        raise KernelError("delta_prep: a section lies outside the projection row")
    pp, ld = _f32_rows(proj, "proj")
    _check(_lib().af_delta_prep(_ptr(out), pp, ld, c_int(off_k), c_int(off_a), c_int(off_w1),
                                _ptr(a_bias, "a_bias", torch.float32), _ptr(w0, "w0", torch.float32),
                                _ptr(w2t, "w2t", torch.float32), c_int(rank), c_int(T), c_int(heads), c_int(dk),
                                c_float(decay_scale), c_float(key_eps), _stream()))


def state_scan(mode: str, out, r, k, v, state, batch, heads: int, dk: int, dv: int, w=None, u=None, au=None,
               decay=None, silu: bool = False) -> None:
    """The recurrence of a matrix state per head over the step's tokens, sequence by sequence, from
    the state that earlier steps left in ``state`` (float32 [slots, heads, dv, dk]; left updated):

    ``decay``: S <- decay[h] S + k v^T, o = S^T r;
    ``delta``: S <- diag(w) S - au (u^T S) + k v^T, o = S^T r (the decay and the removal act on the state before the token);
    ``channel``: S <- diag(w) S + k v^T, o = S^T r (a decay per key channel and token, no removal).

    r, k, w, u, au: float32 rows [T, heads * dk] (column sections allowed), v [T, heads * dv], out float32
    [T, heads * dv].  ``silu``: r, k and v pass through x * sigmoid(x) as they are read.  A step in which
    every sequence brings one token (T == sequences) runs a kernel of its own that stages nothing."""
    if mode not in SCAN_MODES:
        raise KernelError(f"state_scan: unknown mode '{mode}'")
    T = out.shape[0]
    if state.dtype != torch.float32 or tuple(state.shape[1:]) != (heads, dv, dk) or not state.is_contiguous():
        raise KernelError(f"state_scan: state must be contiguous float32 [slots, {heads}, {dv}, {dk}]")
    for t, name, n in ((r, "r", dk), (k, "k", dk), (v, "v", dv), (out, "out", dv)):
        if tuple(t.shape) != (T, heads * n):
            raise KernelError(f"state_scan: {name} must be [{T}, {heads * n}], got {tuple(t.shape)}")
    null = (ctypes.c_void_p(0), c_longlong(0))
    if mode == "delta":
        if w is None or u is None or au is None:
            raise KernelError("state_scan: the delta rule needs w, u and au")
        extra = [_f32_rows(t, n) for t, n in ((w, "w"), (u, "u"), (au, "au"))]
        dec = ctypes.c_void_p(0)
    elif mode == "channel":
        if w is None or tuple(w.shape) != (T, heads * dk):
            raise KernelError(f"state_scan: a decay per key channel and token, [{T}, {heads * dk}]")
        extra = [_f32_rows(w, "w"), null, null]
        dec = ctypes.c_void_p(0)
    else:
        if decay is None or decay.numel() != heads:
            raise KernelError("state_scan: one decay per head")
        extra = [null, null, null]
        dec = _ptr(decay, "decay", torch.float32)
    rp, kp, vp, op = (_f32_rows(t, n) for t, n in ((r, "r"), (k, "k"), (v, "v"), (out, "out")))
    _check(_lib().af_state_scan(c_int(SCAN_MODES[mode]), *rp, *kp, *vp, *extra[0], *extra[1], *extra[2], dec,
                                _ptr(state, "state", torch.float32), *op,
                                _ptr(batch.seq_starts, "seq_starts", torch.int32), _ptr(batch.slots, "slots", torch.int32),
                                c_int(batch.n_seqs), c_int(T), c_int(heads), c_int(dk), c_int(dv), c_int(1 if silu else 0),
                                _stream()))


GATE_ACTS = {"sigmoid": 0, "silu": 1}


def gated_group_norm(y, o, w, gate, group: int, eps: float, gate_act: str = "sigmoid", in_scale: float = 1.0) -> None:
    """y = o' * rsqrt(mean over each group of ``group`` values of o'^2 + eps) * w * act(gate), o' = in_scale * o,
    act the sigmoid or ("silu") the gate times its sigmoid;
    o float32 [T, n] contiguous, gate float32 rows [T, n] (a column section is fine), w float32 [n]."""
    T, n = o.shape
    if o.dtype != torch.float32 or not o.is_contiguous() or tuple(y.shape) != (T, n) or not y.is_contiguous():
        raise KernelError("gated_group_norm: o float32 and y, both contiguous [T, n]")
    if w.numel() != n or tuple(gate.shape) != (T, n):
        raise KernelError("gated_group_norm: weight [n] and gate [T, n]")
    gp, gts = _f32_rows(gate, "gate")
    _check(_lib().af_gated_group_norm(_ptr(y), c_int(dtype_code(y.dtype)), _ptr(o), _ptr(w, "w", torch.float32), gp, gts,
                                      c_int(T), c_int(n), c_int(group), c_float(eps), c_int(GATE_ACTS[gate_act]),
                                      c_float(in_scale), _stream()))


def gated_scan(y, proj, off_z: int, off_x: int, off_g: int, bz, bx, state, batch) -> None:
    """A gated recurrence over a vector state, channel by channel: with the sections z, x, g of the packed
    float32 projection rows, gate = sigmoid(z + bz), c = x + bx, candidate = c + 1/2 where c >= 0 and
    sigmoid(c) below, S <- (1 - gate) S + gate * candidate, y = S * silu(g).  ``state`` float32
    [slots, width] is read and left updated."""
    T, width = y.shape
    if not y.is_contiguous() or state.dtype != torch.float32 or tuple(state.shape[1:]) != (width,) \
            or not state.is_contiguous():
        raise KernelError(f"gated_scan: y contiguous [T, {width}], state contiguous float32 [slots, {width}]")
    if max(off_z, off_x, off_g) + width > proj.shape[1] or bz.numel() != width or bx.numel() != width:
        raise KernelError("gated_scan: a section lies outside the projection row, or a bias of another size")
    pp, ld = _f32_rows(proj, "proj")
    _check(_lib().af_gated_scan(_ptr(y), c_int(dtype_code(y.dtype)), pp, ld, c_int(off_z), c_int(off_x), c_int(off_g),
                                _ptr(bz, "bz", torch.float32), _ptr(bx, "bx", torch.float32),
                                _ptr(state, "state", torch.float32), _ptr(batch.seq_starts, "seq_starts", torch.int32),
                                _ptr(batch.slots, "slots", torch.int32), c_int(batch.n_seqs), c_int(width), _stream()))


def qk_norm_rope_store(qkv, proj, batch, nq: int, nkv: int, hd: int, inv_freq, rot_dim: int, pairing: str,
                       q_weight=None, k_weight=None, eps: float = 0.0, v_from_k: bool = False, kv=None,
                       bias=None, norm_after: bool = False, magnitude: float = 1.0, dv=None, pitch: int = 0,
                       whole_norm: bool = False, table=None) -> None:
    """From float32 projection rows [q heads | k heads (| v heads of ``dv`` values)], plus ``bias`` (float32,
    laid out like a row) when given: q and k heads normalised per head
    (x * rsqrt(mean x^2 + eps) * weight, the weight of ``hd`` values shared by the heads; no weights: as
    they are), their first ``rot_dim`` elements rotated (cosines and sines times ``magnitude``), with
    ``norm_after`` divided by their root mean square over the head after that (eps inside the root, no weight),
    into the packed rows ``qkv`` [q | k | v] of the
    compute dtype; the value heads are the raw k heads of the projection (``v_from_k``) or the projection's own.
    With ``kv`` (the layer's view of its cache pages) k and v also go to each token's row of its page.
    ``pitch`` > 0: every head of ``qkv`` and every row of the cache holds that many elements (at least ``hd`` and
    ``dv``), zeros behind its own.  ``whole_norm``: q (and k) are normalised over the token's whole projection, all
    heads at once, and the weights hold ``nq * hd`` and ``nkv * hd`` values.  ``table`` (float32 [T, rot_dim / 2,
    2]): the step's cosines and sines, taken instead of working them out from ``inv_freq``."""
    if table is not None and (tuple(table.shape) != (proj.shape[0], rot_dim // 2, 2) or table.dtype != torch.float32
                              or not table.is_contiguous()):
        raise KernelError(f"qk_norm_rope_store: a table of cosines and sines [{proj.shape[0]}, {rot_dim // 2}, 2]")
    T = proj.shape[0]
    dv = dv or hd
    pk, pv = (pitch, pitch) if pitch else (hd, dv)
    if pitch and (pitch < hd or pitch < dv):
        raise KernelError(f"qk_norm_rope_store: a pitch of {pitch} below the heads' {hd} and {dv}")
    width_in = (nq + nkv) * hd if v_from_k else (nq + nkv) * hd + nkv * dv
    if proj.shape[1] < width_in or tuple(qkv.shape) != (T, (nq + nkv) * pk + nkv * pv):
        raise KernelError(f"qk_norm_rope_store: projection of {width_in} columns into rows of {(nq + nkv) * pk + nkv * pv}")
    if pairing not in PAIRINGS or inv_freq.numel() != rot_dim // 2:
        raise KernelError("qk_norm_rope_store: pairing, or inv_freq does not hold rot_dim / 2 values")
    for wgt, heads in ((q_weight, nq), (k_weight, nkv)):
        want = heads * hd if whole_norm else hd
        if (wgt is None and whole_norm) or (wgt is not None and wgt.numel() != want):
            raise KernelError(f"qk_norm_rope_store: a norm weight of {want} values")
    if bias is not None and bias.numel() < width_in:
        raise KernelError(f"qk_norm_rope_store: a bias of {width_in} values")
    kc = vc = pt = None
    max_pages = ring = 0
    if kv is not None:
        kc, vc, pt, ring = kv.k, kv.v, kv.page_table, kv.ring_rows
        if kc.dtype != qkv.dtype or tuple(kc.shape[1:]) != (nkv, PAGE, pk) or vc is None \
                or tuple(vc.shape[1:]) != (nkv, PAGE, pv) or not kc.is_contiguous() or not vc.is_contiguous():
            raise KernelError(f"qk_norm_rope_store: cache pages must be [pages, {nkv}, {PAGE}, {pk}] (values {pv}) "
                              "of the rows' dtype")
        max_pages = pt.shape[1]
    pp, ld = _f32_rows(proj, "proj")
    _check(_lib().af_qk_norm_rope_store(
        _ptr(qkv), c_int(dtype_code(qkv.dtype)), c_longlong(_rows(qkv, "qkv")), pp, ld,
        _ptr(bias, "bias", torch.float32, allow_none=True),
        _ptr(q_weight, "q_weight", torch.float32, allow_none=True),
        _ptr(k_weight, "k_weight", torch.float32, allow_none=True), c_float(eps), c_int(1 if norm_after else 0),
        c_float(magnitude), c_int(1 if v_from_k else 0),
        _ptr(batch.positions, "positions", torch.int32), _ptr(batch.seq_of_token, "seq_of_token", torch.int32),
        _ptr(batch.slots, "slots", torch.int32), _ptr(batch.len_after, "len_after", torch.int32),
        _ptr(inv_freq, "inv_freq", torch.float32), _ptr(table, "table", torch.float32, allow_none=True),
        c_int(T), c_int(nq), c_int(nkv), c_int(hd), c_int(dv), c_int(rot_dim),
        c_int(PAIRINGS[pairing]), _ptr(kc, allow_none=True), _ptr(vc, allow_none=True),
        _ptr(pt, "page_table", torch.int32, allow_none=True), c_int(max_pages), c_int(ring), c_int(pitch),
        c_int(1 if whole_norm else 0), _stream()))


def attn_prefill_fast_head(size: int) -> int:
    """The smallest head size that a bfloat16 tensor-core prefill kernel takes and that holds ``size`` elements
    (a mixer may pad its heads with zeros up to it), or 0."""
    for hd in (64, 128, 256):
        if hd >= size and (_lib().af_attn_prefill_tc_supported(c_int(hd)) or _lib().af_attn_prefill_supported(c_int(hd))):
            return hd
    return 0


def latent_prep(q, kvrow, proj, batch, heads: int, dim: int, rot: int, rank: int, norm_w, eps: float, inv_freq,
                kv=None, pitch: int = 0) -> None:
    """From float32 projection rows [q heads of (dim + rot) | latent of ``rank`` | shared key part of ``rot``]:
    the q heads with their last ``rot`` elements rotated (pairs i, i + rot / 2) into ``q`` [T, heads pitch]
    (``pitch`` >= dim + rot, by default that: a head's elements beyond dim + rot are set to zero);
    the latent over its root mean square (eps inside the root) times ``norm_w`` and the rotated shared key part
    into ``kvrow`` [T, rank + rot], and, with ``kv`` (the layer's view of its cache: one kv head of rank + rot
    elements, no value pages), into each token's row of its page."""
    T = proj.shape[0]
    pitch = pitch or dim + rot
    if proj.shape[1] < heads * (dim + rot) + rank + rot or tuple(q.shape) != (T, heads * pitch) \
            or tuple(kvrow.shape) != (T, rank + rot) or q.dtype != kvrow.dtype:
        raise KernelError("latent_prep: shapes of the projection, q and kv rows do not fit")
    if inv_freq.numel() != rot // 2 or norm_w.numel() != rank:
        raise KernelError("latent_prep: inv_freq holds rot / 2 values, the norm weight rank values")
    kc = pt = None
    max_pages = ring = 0
    if kv is not None:
        kc, pt, ring = kv.k, kv.page_table, kv.ring_rows
        if kc.dtype != q.dtype or tuple(kc.shape[1:]) != (1, PAGE, rank + rot) or not kc.is_contiguous():
            raise KernelError(f"latent_prep: cache pages must be [pages, 1, {PAGE}, {rank + rot}] of the rows' dtype")
        max_pages = pt.shape[1]
    pp, ld = _f32_rows(proj, "proj")
    _check(_lib().af_latent_prep(
        _ptr(q), c_longlong(_rows(q, "q")), _ptr(kvrow), c_longlong(_rows(kvrow, "kvrow")), c_int(dtype_code(q.dtype)),
        pp, ld, _ptr(norm_w, "norm_w", torch.float32), c_float(eps), _ptr(batch.positions, "positions", torch.int32),
        _ptr(batch.seq_of_token, "seq_of_token", torch.int32), _ptr(batch.slots, "slots", torch.int32),
        _ptr(batch.len_after, "len_after", torch.int32), _ptr(inv_freq, "inv_freq", torch.float32), c_int(T),
        c_int(heads), c_int(dim), c_int(rot), c_int(rank), c_int(pitch), _ptr(kc, allow_none=True),
        _ptr(pt, "page_table", torch.int32, allow_none=True), c_int(max_pages), c_int(ring), _stream()))


def head_project(out, x, w, heads: int, D: int, N: int, extra: int = 0, x_pitch: int = 0) -> None:
    """out[t, h, :N] = x[t, h, :D] @ w[h] for w [heads, D, N] (32-bit sums), and the ``extra`` elements behind a
    head's D inputs copied behind its N outputs.  x [T, heads x_pitch] (``x_pitch`` = D + extra by default: what
    else a head holds is skipped), out [T, heads (N + extra)]: row views of one dtype, which is w's too."""
    T = x.shape[0]
    x_pitch = x_pitch or D + extra
    if tuple(x.shape) != (T, heads * x_pitch) or tuple(out.shape) != (T, heads * (N + extra)) \
            or tuple(w.shape) != (heads, D, N) or not w.is_contiguous() or not (x.dtype == out.dtype == w.dtype):
        raise KernelError("head_project: shapes or dtypes do not fit")
    _check(_lib().af_head_project(_ptr(out), c_longlong(_rows(out, "out")), _ptr(x), c_longlong(_rows(x, "x")), _ptr(w),
                                  c_int(dtype_code(x.dtype)), c_int(T), c_int(heads), c_int(D), c_int(N), c_int(extra),
                                  c_int(x_pitch), _stream()))


# ---------------------------------------------------------------- the norm without statistics, and re-entry

def tanh_norm(y, x, w, b, alpha: float, rows=None) -> None:
    """y = tanh(alpha x) w + b (32-bit), of the listed rows of x when ``rows`` is given."""
    n, H = y.shape
    if not y.is_contiguous() or not x.is_contiguous() or x.shape[1] != H or w.numel() != H or b.numel() != H:
        raise KernelError("tanh_norm: shapes do not fit")
    if rows is None and x.shape[0] != n:
        raise KernelError("tanh_norm: as many rows out as in")
    _check(_lib().af_tanh_norm(_ptr(y), c_int(dtype_code(y.dtype)), _ptr(x, "x", torch.float32),
                               _ptr(w, "w", torch.float32), _ptr(b, "b", torch.float32), c_float(alpha),
                               _ptr(rows, "rows", torch.int32, allow_none=True), c_int(n), c_int(H), _stream()))


def add_tanh_norm(x, a, w, b, alpha: float, y=None, w_next=None, b_next=None, alpha_next: float = 0.0) -> None:
    """x += tanh(alpha a) w + b in place (32-bit); ``a`` [rows, H] of the compute dtype or float32, or float32
    partial sums [n, rows, H] added in index order first.  With ``y``: also y = tanh(alpha_next x) w_next + b_next."""
    n, H = x.shape
    parts = a.shape[0] if a.dim() == 3 else 1
    if not x.is_contiguous() or not a.is_contiguous() or tuple(a.shape[-2:]) != (n, H) or (y is not None and not y.is_contiguous()):
        raise KernelError("add_tanh_norm: shapes do not fit")
    _check(_lib().af_add_tanh_norm(
        _ptr(x, "x", torch.float32), _ptr(a), c_int(dtype_code(a.dtype)), c_int(parts), c_longlong(n * H),
        _ptr(w, "w", torch.float32), _ptr(b, "b", torch.float32), c_float(alpha), _ptr(y, "y", allow_none=True),
        c_int(dtype_code(y.dtype) if y is not None else F32), _ptr(w_next, "w_next", torch.float32, allow_none=True),
        _ptr(b_next, "b_next", torch.float32, allow_none=True), c_float(alpha_next), c_int(n), c_int(H), _stream()))


def concat_cast(out, a, b) -> None:
    """out = [a | b] row by row in out's dtype; a and b float32."""
    n = out.shape[0]
    if tuple(out.shape) != (n, a.shape[1] + b.shape[1]) or a.shape[0] != n or b.shape[0] != n \
            or not (out.is_contiguous() and a.is_contiguous() and b.is_contiguous()):
        raise KernelError("concat_cast: shapes do not fit")
    _check(_lib().af_concat_cast(_ptr(out), c_int(dtype_code(out.dtype)), _ptr(a, "a", torch.float32),
                                 _ptr(b, "b", torch.float32), c_int(n), c_int(a.shape[1]), c_int(b.shape[1]), _stream()))


def set_sum_row(x, z, row, y=None, w=None, b=None, alpha: float = 0.0) -> None:
    """x = z + row for every row (z [rows, H], or float32 partial sums [n, rows, H] added in index order; ``row``
    float32 [H]); with ``y``: also y = tanh(alpha x) w + b."""
    n, H = x.shape
    parts = z.shape[0] if z.dim() == 3 else 1
    if not x.is_contiguous() or not z.is_contiguous() or tuple(z.shape[-2:]) != (n, H) or row.numel() != H:
        raise KernelError("set_sum_row: shapes do not fit")
    _check(_lib().af_set_sum_row(
        _ptr(x, "x", torch.float32), _ptr(z), c_int(dtype_code(z.dtype)), c_int(parts), c_longlong(n * H),
        _ptr(row, "row", torch.float32), _ptr(y, "y", allow_none=True),
        c_int(dtype_code(y.dtype) if y is not None else F32), _ptr(w, "w", torch.float32, allow_none=True),
        _ptr(b, "b", torch.float32, allow_none=True), c_float(alpha), c_int(n), c_int(H), _stream()))


def add_scaled_rmsnorm(x, terms, y=None, w_next=None, eps: float = 0.0, offset: float = 0.0) -> None:
    """x += sum of scale * term over ``terms`` (a list of (tensor, scale): a tensor [rows, H] of the
    compute dtype, or float32 partial sums [n, rows, H], added in index order); then, when ``y`` is
    given, y = norm(x) * (offset + w_next).  Two terms a kernel; the norm rides on the last."""
    n, H = x.shape
    if not x.is_contiguous() or (y is not None and not y.is_contiguous()):
        raise KernelError("add_scaled_rmsnorm: tensors must be contiguous")
    if not terms:
        raise KernelError("add_scaled_rmsnorm: at least one term")

    def arg(t):
        parts = 1
        if t.dim() == 3:
            parts = t.shape[0]
            if t.dtype != torch.float32:
                raise KernelError("add_scaled_rmsnorm: partial sums are float32")
        if tuple(t.shape[-2:]) != (n, H) or not t.is_contiguous():
            raise KernelError(f"add_scaled_rmsnorm: a term of shape {tuple(t.shape)} for rows {(n, H)}")
        return _ptr(t), c_int(dtype_code(t.dtype)), c_int(parts)

    for i in range(0, len(terms), 2):
        pair = terms[i:i + 2]
        last = i + 2 >= len(terms)
        a, sa = pair[0]
        b, sb = pair[1] if len(pair) > 1 else (None, 0.0)
        barg = arg(b) if b is not None else (ctypes.c_void_p(0), c_int(F32), c_int(1))
        yy = y if last else None
        _check(_lib().af_add_scaled_rmsnorm(
            _ptr(x, "x", torch.float32), *arg(a), c_float(sa), *barg, c_float(sb), _ptr(yy, "y", allow_none=True),
            c_int(dtype_code(yy.dtype) if yy is not None else F32),
            _ptr(w_next, "w_next", torch.float32, allow_none=True) if yy is not None else ctypes.c_void_p(0),
            c_int(n), c_int(H), c_float(eps), c_float(offset), _stream()))


def _term_arg(t, n: int, H: int, who: str):
    """Pointer, dtype code and number of partial sums of one term of a sum (a tensor [rows, H] of the
    compute dtype or float32, or float32 partial sums [n, rows, H])."""
    parts = 1
    if t.dim() == 3:
        parts = t.shape[0]
        if t.dtype != torch.float32:
            raise KernelError(f"{who}: partial sums are float32")
    if tuple(t.shape[-2:]) != (n, H) or not t.is_contiguous():
        raise KernelError(f"{who}: a term of shape {tuple(t.shape)} for rows {(n, H)}")
    return _ptr(t), c_int(dtype_code(t.dtype)), c_int(parts)


def add_normed_terms(x, terms, w_post, eps_post: float, offset_post: float = 0.0, y=None, w_next=None,
                     eps_next: float = 0.0, offset_next: float = 0.0) -> None:
    """x += norm(sum of scale * term) * (offset_post + w_post): the sum of the ``terms`` (as in
    :func:`add_scaled_rmsnorm`) and the norm's statistics in 32 bits.  With ``y``: y = norm(x) *
    (offset_next + w_next), or without ``w_next`` the new x itself in y's dtype.  More than two terms are
    first added into a float32 row of their own."""
    n, H = x.shape
    if not x.is_contiguous() or (y is not None and not y.is_contiguous()):
        raise KernelError("add_normed_terms: tensors must be contiguous")
    if not terms:
        raise KernelError("add_normed_terms: at least one term")
    if len(terms) > 2:
        total = torch.zeros(n, H, dtype=torch.float32, device=x.device)
        add_scaled_rmsnorm(total, terms)
        terms = [(total, 1.0)]
    a, sa = terms[0]
    b, sb = terms[1] if len(terms) > 1 else (None, 0.0)
    barg = _term_arg(b, n, H, "add_normed_terms") if b is not None else (ctypes.c_void_p(0), c_int(F32), c_int(1))
    _check(_lib().af_add_normed_terms(
        _ptr(x, "x", torch.float32), *_term_arg(a, n, H, "add_normed_terms"), c_float(sa), *barg, c_float(sb),
        _ptr(w_post, "w_post", torch.float32), c_float(eps_post), c_float(offset_post), _ptr(y, "y", allow_none=True),
        c_int(dtype_code(y.dtype) if y is not None else F32), _ptr(w_next, "w_next", torch.float32, allow_none=True),
        c_float(eps_next), c_float(offset_next), c_int(n), c_int(H), _stream()))


def cast_rows(y, x, rows=None) -> None:
    """y[r] = x[rows[r]] (or x[r]) in y's dtype; x float32 [T, H]."""
    n, H = y.shape
    if not (x.is_contiguous() and y.is_contiguous()) or x.shape[1] != H:
        raise KernelError("cast_rows: contiguous tensors of one row size")
    _check(_lib().af_cast_rows(_ptr(y, "y"), c_int(dtype_code(y.dtype)), _ptr(x, "x", torch.float32),
                               _ptr(rows, "rows", torch.int32, allow_none=True), c_int(n), c_int(H), _stream()))


def scale_(z, s: float) -> None:
    """z *= s (float32, in place)."""
    if not z.is_contiguous():
        raise KernelError("scale_: tensor must be contiguous")
    _check(_lib().af_scale(_ptr(z, "z", torch.float32), c_longlong(z.numel()), c_float(s), _stream()))


# ---------------------------------------------------------------- a gated linear recurrence with a convolution in front

def conv_rows(u, proj, off_x: int, bx, cw, cb, state, batch, u16=None) -> None:
    """u = the causal convolution per channel of (section ``off_x`` of the float32 projection rows + bx), plus
    cb: ``cw`` float32 [taps, width] (the stored taps transposed), the last tap on the current token; the tokens before the step come from
    rows 1 .. taps-1 of the sequence's ``state`` (float32 [slots, taps, width]; zeros for a new sequence).
    ``u16`` (bfloat16, like u): also receives u, rounded."""
    T, width = u.shape
    if u16 is not None and (u16.dtype != torch.bfloat16 or u16.shape != u.shape or not u16.is_contiguous()):
        raise KernelError("conv_rows: u16 is a contiguous bfloat16 tensor of u's shape")
    taps = cw.shape[0]
    if u.dtype != torch.float32 or not u.is_contiguous() or tuple(cw.shape) != (taps, width) or not cw.is_contiguous():
        raise KernelError(f"conv_rows: u contiguous float32 [T, {width}], taps [taps, {width}]")
    if tuple(state.shape[1:]) != (taps, width) or state.dtype != torch.float32 or not state.is_contiguous():
        raise KernelError(f"conv_rows: state must be contiguous float32 [slots, {taps}, {width}]")
    if off_x + width > proj.shape[1] or bx.numel() != width or cb.numel() != width:
        raise KernelError("conv_rows: the section lies outside the projection row, or a bias of another size")
    pp, ld = _f32_rows(proj, "proj")
    _check(_lib().af_conv_rows(_ptr(u), _ptr(u16, allow_none=True), pp, ld, c_int(off_x), _ptr(bx, "bx", torch.float32), _ptr(cw, "cw", torch.float32),
                               _ptr(cb, "cb", torch.float32), _ptr(state, "state", torch.float32),
                               _ptr(batch.seq_of_token, "seq_of_token", torch.int32),
                               _ptr(batch.seq_starts, "seq_starts", torch.int32), _ptr(batch.slots, "slots", torch.int32),
                               c_int(T), c_int(width), c_int(taps), _stream()))


def gate_rows(decay, inp, u, wa, wi, ba, bi, rate) -> None:
    """With the channels of u (float32 [T, width]) in ``blocks`` equal parts and wa, wi [blocks, out, in]:
    r = sigmoid(wa_b u_b + ba), i = sigmoid(wi_b u_b + bi), a = exp(-rate r), decay = 1 - a, inp = sqrt(1 - a^2) i u
    (all float32 [T, width]; the weights may be of the compute dtype, the sums are 32-bit)."""
    T, width = u.shape
    blocks, bw = wa.shape[0], wa.shape[1]
    if blocks * bw != width or tuple(wa.shape) != (blocks, bw, bw) or wi.shape != wa.shape or wi.dtype != wa.dtype \
            or not (wa.is_contiguous() and wi.is_contiguous()):
        raise KernelError(f"gate_rows: gate matrices [blocks, {width} / blocks, {width} / blocks] of one dtype")
    for t, name in ((decay, "decay"), (inp, "inp"), (u, "u")):
        if t.dtype != torch.float32 or tuple(t.shape) != (T, width) or not t.is_contiguous():
            raise KernelError(f"gate_rows: {name} must be contiguous float32 [{T}, {width}]")
    if ba.numel() != width or bi.numel() != width or rate.numel() != width:
        raise KernelError("gate_rows: biases and rates of one value a channel")
    _check(_lib().af_gate_rows(_ptr(decay), _ptr(inp), _ptr(u), _ptr(wa), _ptr(wi), c_int(dtype_code(wa.dtype)),
                               _ptr(ba, "ba", torch.float32), _ptr(bi, "bi", torch.float32),
                               _ptr(rate, "rate", torch.float32), c_int(T), c_int(width), c_int(blocks), _stream()))


GATE_TC_ROWS = 64     # from so many rows on the gates' products go to the tensor cores


def gate_rows_tc_supported(u, wa) -> bool:
    """Whether :func:`gate_rows_tc` takes these: bfloat16 matrices whose blocks hold a multiple of 8 channels."""
    return wa.dtype == torch.bfloat16 and wa.shape[1] % 8 == 0 and wa.is_contiguous() and wa.data_ptr() % 16 == 0


def gate_rows_tc(decay, inp, u, u16, wa, wi, ba, bi, rate) -> None:
    """:func:`gate_rows` with the two products on the tcgen05 tensor cores: they read ``u16``, the bfloat16
    rounding of u (bfloat16 matrices, 32-bit sums); the sigmoids, the decay and the input of the scan are worked
    out in 32 bits from the sums and the 32-bit u."""
    T, width = u.shape
    blocks, bw = wa.shape[0], wa.shape[1]
    if blocks * bw != width or tuple(wa.shape) != (blocks, bw, bw) or wi.shape != wa.shape or wi.dtype != wa.dtype \
            or not gate_rows_tc_supported(u, wa) or not wi.is_contiguous() or wi.data_ptr() % 16:
        raise KernelError(f"gate_rows_tc: bfloat16 gate matrices [blocks, {width} / blocks, {width} / blocks], blocks of a multiple of 8")
    for t, name in ((decay, "decay"), (inp, "inp"), (u, "u")):
        if t.dtype != torch.float32 or tuple(t.shape) != (T, width) or not t.is_contiguous():
            raise KernelError(f"gate_rows_tc: {name} must be contiguous float32 [{T}, {width}]")
    if u16.dtype != torch.bfloat16 or u16.shape != u.shape or not u16.is_contiguous() or u16.data_ptr() % 16:
        raise KernelError("gate_rows_tc: u16 is u in bfloat16")
    if ba.numel() != width or bi.numel() != width or rate.numel() != width:
        raise KernelError("gate_rows_tc: biases and rates of one value a channel")
    _check(_lib().af_gate_rows_tc(_ptr(decay), _ptr(inp), _ptr(u), _ptr(u16), _ptr(wa), _ptr(wi),
                                  _ptr(ba, "ba", torch.float32), _ptr(bi, "bi", torch.float32),
                                  _ptr(rate, "rate", torch.float32), c_int(T), c_int(blocks), c_int(bw),
                                  _ptr(error_word(u.device), "err", torch.int32), _stream()))


def decay_scan(out, decay, inp, proj, off_y: int, off_x: int, by, bx, state, batch) -> None:
    """S <- S - decay S + inp (``decay`` = 1 - a) token after token from row 0 of the sequence's ``state`` (float32 [slots, taps, width];
    left updated, with the last taps - 1 values of section ``off_x`` + bx in the rows behind it);
    out = S * gelu_tanh(section ``off_y`` of the projection rows + by)."""
    T, width = out.shape
    taps = state.shape[1]
    if not out.is_contiguous() or state.dtype != torch.float32 or tuple(state.shape[1:]) != (taps, width) \
            or not state.is_contiguous():
        raise KernelError(f"decay_scan: out contiguous [T, {width}], state contiguous float32 [slots, taps, {width}]")
    for t, name in ((decay, "decay"), (inp, "inp")):
        if t.dtype != torch.float32 or tuple(t.shape) != (T, width) or not t.is_contiguous():
            raise KernelError(f"decay_scan: {name} must be contiguous float32 [{T}, {width}]")
    if max(off_y, off_x) + width > proj.shape[1] or by.numel() != width or bx.numel() != width:
        raise KernelError("decay_scan: a section lies outside the projection row, or a bias of another size")
    pp, ld = _f32_rows(proj, "proj")
    _check(_lib().af_decay_scan(_ptr(out), c_int(dtype_code(out.dtype)), _ptr(decay), _ptr(inp), pp, ld, c_int(off_y),
                                c_int(off_x), _ptr(by, "by", torch.float32), _ptr(bx, "bx", torch.float32),
                                _ptr(state, "state", torch.float32), _ptr(batch.seq_starts, "seq_starts", torch.int32),
                                _ptr(batch.slots, "slots", torch.int32), c_int(batch.n_seqs), c_int(out.shape[0]), c_int(width),
                                c_int(taps), _stream()))


# ---------------------------------------------------------------- routed experts

EXPERT_TILE = 32     # pairs of one expert that a block of the experts' products on the CUDA cores takes
EXPERT_TC_TILES = (16, 32, 64, 128, 256)     # row tiles of the products on the tensor cores


def expert_max_tiles(n_pairs: int, n_experts: int, tile: int = EXPERT_TILE) -> int:
    """Room for the tiles of ``n_pairs`` (token, choice) pairs however they fall on the experts."""
    return min(n_pairs, n_pairs // tile + n_experts)


def expert_tc_tile(n_pairs: int, n_experts: int) -> int:
    """The row tile of the tensor-core products: the smallest that holds an expert's share of the pairs when
    they fall evenly (an expert with more gets several tiles of equal size)."""
    share = (n_pairs + n_experts - 1) // n_experts
    return next((t for t in EXPERT_TC_TILES if t >= share), EXPERT_TC_TILES[-1])


def expert_route(ids, wts, shared_gate, h, router, n_experts: int, correction=None, groups: int = 1, keep: int = 1,
                 normalise: bool = False, out_scale: float = 1.0) -> None:
    """Per row of h [T, H]: scores = sigmoid(router[:n_experts] h) in 32 bits; ids, wts [T, top] = the experts
    with the largest scores (equal scores: the lower index) and their scores; ``shared_gate`` float32 [T], when
    given, = sigmoid(router[n_experts] h).  ``correction`` (float32 [experts]) is added to the scores for the
    choice only.  ``groups`` > 1: the experts form so many equal groups of neighbours, a group's score is the sum
    of its two largest choice scores, and only experts of the ``keep`` best groups can be chosen.  ``normalise``:
    the chosen scores are divided by their sum + 1e-20; ``out_scale`` multiplies the weights."""
    T, H = h.shape
    top = ids.shape[1]
    rows = n_experts + (1 if shared_gate is not None else 0)
    if tuple(router.shape) != (rows, H) or router.dtype != torch.float32 or not router.is_contiguous():
        raise KernelError(f"expert_route: router must be contiguous float32 [{rows}, {H}]")
    if tuple(ids.shape) != (T, top) or tuple(wts.shape) != (T, top) or not (ids.is_contiguous() and wts.is_contiguous()
                                                                           and h.is_contiguous()):
        raise KernelError("expert_route: ids and wts contiguous [T, top], h contiguous")
    if correction is not None and (correction.numel() != n_experts or not correction.is_contiguous()):
        raise KernelError(f"expert_route: a correction of {n_experts} values")
    scores = torch.empty(T, rows, dtype=torch.float32, device=h.device)      # (between the two kernels)
    _check(_lib().af_expert_route(_ptr(ids, "ids", torch.int32), _ptr(wts, "wts", torch.float32),
                                  _ptr(shared_gate, "shared_gate", torch.float32, allow_none=True), _ptr(scores), _ptr(h),
                                  c_int(dtype_code(h.dtype)), _ptr(router), c_int(T), c_int(H), c_int(n_experts),
                                  c_int(top), _ptr(correction, "correction", torch.float32, allow_none=True),
                                  c_int(groups), c_int(keep if groups > 1 else 1), c_int(1 if normalise else 0),
                                  c_float(out_scale), _stream()))


def expert_plan(perm, plan, ids, n_experts: int, tile: int = EXPERT_TILE) -> None:
    """The (token, choice) pairs of ``ids`` [T, top] sorted by expert: perm int32 [T * top] (sorted row -> pair),
    plan int32 [1 + 3 * expert_max_tiles]: tiles in use, then (expert, first sorted row, rows) per tile; a tile
    holds up to ``tile`` rows, and an expert's tiles are of equal size."""
    n_pairs = ids.numel()
    max_tiles = (plan.numel() - 1) // 3
    if perm.numel() != n_pairs or not (perm.is_contiguous() and plan.is_contiguous() and ids.is_contiguous()):
        raise KernelError("expert_plan: one entry of perm per pair")
    _check(_lib().af_expert_plan(_ptr(perm, "perm", torch.int32), _ptr(plan, "plan", torch.int32),
                                 _ptr(ids, "ids", torch.int32), c_int(n_pairs), c_int(n_experts), c_int(max_tiles),
                                 c_int(tile), _stream()))


EXPERT_ACTS = {None: 0, "gelu_erf": 1}


def expert_rows(out, a, w0, w1=None, perm=None, plan=None, pair_weight=None, scale_out=None, n_tokens: int = 0,
                top: int = 1, limit: float = 0.0, act=None) -> None:
    """Rows times the matrices of the expert they belong to (the CUDA-core path; 32-bit sums in index order).
    With ``w1``: out[sorted row] = act(s x w0[e]^T, s x w1[e]^T) * post in the compute dtype, x = row
    pair // top of ``a``, s = pair_weight[pair], post = scale_out[token], act(g, u) = min(g, limit)
    sigmoid(1.702 min(g, limit)) (clamp(u, +-limit) + 1).  Without: out float32 [top, tokens, N] with
    out[choice, token] = a[sorted row] w0[e]^T.  Without ``w1`` but with ``act`` = "gelu_erf": an expert of one
    matrix, out[sorted row] = gelu(x w0[e]^T) * s * post with the exact GELU (the weight stands behind the
    activation).  w0, w1: [experts, N, K].  Without a plan: one expert, the rows in order."""
    n_rows = n_tokens * top
    E, N, K = w0.shape
    if not (a.is_contiguous() and out.is_contiguous() and w0.is_contiguous()) or a.shape[1] != K or a.dtype != w0.dtype:
        raise KernelError("expert_rows: contiguous rows of the matrices' dtype and row size")
    if act not in EXPERT_ACTS or (act is not None and w1 is not None):
        raise KernelError(f"expert_rows: activation '{act}' (known: gelu_erf, behind one matrix)")
    if w1 is not None or act is not None:
        if w1 is not None and (w1.shape != w0.shape or w1.dtype != w0.dtype or not w1.is_contiguous()):
            raise KernelError("expert_rows: gate and up matrices alike")
        if tuple(out.shape) != (n_rows, N) or out.dtype != a.dtype or a.shape[0] != n_tokens:
            raise KernelError(f"expert_rows: out [{n_rows}, {N}] of the rows' dtype")
    elif tuple(out.shape) != (top, n_tokens, N) or out.dtype != torch.float32 or a.shape[0] != n_rows:
        raise KernelError(f"expert_rows: out float32 [{top}, {n_tokens}, {N}] from {n_rows} rows")
    if plan is None and E != 1:
        raise KernelError("expert_rows: several experts need a plan")
    max_tiles = (plan.numel() - 1) // 3 if plan is not None else 0
    _check(_lib().af_expert_rows(_ptr(out), _ptr(a), _ptr(w0), _ptr(w1, allow_none=True), c_int(dtype_code(a.dtype)),
                                 _ptr(perm, "perm", torch.int32, allow_none=True),
                                 _ptr(plan, "plan", torch.int32, allow_none=True),
                                 _ptr(pair_weight, "pair_weight", torch.float32, allow_none=True),
                                 _ptr(scale_out, "scale_out", torch.float32, allow_none=True), c_int(n_rows),
                                 c_int(n_tokens), c_int(top), c_int(max_tiles), c_int(N), c_int(K), c_float(limit),
                                 c_int(EXPERT_ACTS[act]), _stream()))


def expert_gather(out, x, perm, top: int) -> None:
    """out[sorted row] = x[perm[sorted row] // top]: the tokens' rows in the order of the plan."""
    n_rows, H = out.shape
    if not (out.is_contiguous() and x.is_contiguous()) or x.shape[1] != H or out.dtype != x.dtype \
            or perm.numel() != n_rows or x.shape[0] * top != n_rows:
        raise KernelError("expert_gather: contiguous rows of one size and dtype, one entry of perm a row")
    _check(_lib().af_expert_gather(_ptr(out), _ptr(x), c_int(dtype_code(x.dtype)), _ptr(perm, "perm", torch.int32),
                                   c_int(n_rows), c_int(top), c_int(H), _stream()))


def expert_rows_tc_supported(a, w0) -> bool:
    """Whether the tensor-core products take these rows and matrices: bfloat16, contiguous, K a multiple of 8,
    16-byte aligned."""
    return (a.dtype == torch.bfloat16 and w0.dtype == torch.bfloat16 and a.is_contiguous() and w0.is_contiguous()
            and a.shape[1] % 8 == 0 and a.data_ptr() % 16 == 0 and w0.data_ptr() % 16 == 0)


def expert_rows_tc(out, a, w0, w1=None, perm=None, plan=None, pair_weight=None, scale_out=None, n_tokens: int = 0,
                   top: int = 1, limit: float = 0.0, tile: int = 0, act=None) -> None:
    """:func:`expert_rows` on the tcgen05 tensor cores (bfloat16 operands, 32-bit sums in TMEM), with one
    difference: ``a`` holds the sorted rows themselves also for the first product (:func:`expert_gather`).
    ``tile``: the row tile the plan was made for (without a plan: chosen here)."""
    n_rows = n_tokens * top
    E, N, K = w0.shape
    if not expert_rows_tc_supported(a, w0) or tuple(a.shape) != (n_rows, K) or not out.is_contiguous():
        raise KernelError("expert_rows_tc: contiguous bfloat16 rows [rows, K], K a multiple of 8, 16-byte aligned")
    if act not in EXPERT_ACTS or (act is not None and w1 is not None):
        raise KernelError(f"expert_rows_tc: activation '{act}' (known: gelu_erf, behind one matrix)")
    if w1 is not None or act is not None:
        if w1 is not None and (w1.shape != w0.shape or w1.dtype != w0.dtype or not w1.is_contiguous() or w1.data_ptr() % 16):
            raise KernelError("expert_rows_tc: gate and up matrices alike")
        if tuple(out.shape) != (n_rows, N) or out.dtype != torch.bfloat16:
            raise KernelError(f"expert_rows_tc: out bfloat16 [{n_rows}, {N}]")
    elif tuple(out.shape) != (top, n_tokens, N) or out.dtype != torch.float32:
        raise KernelError(f"expert_rows_tc: out float32 [{top}, {n_tokens}, {N}]")
    if plan is None:
        if E != 1:
            raise KernelError("expert_rows_tc: several experts need a plan")
        tile = expert_tc_tile(n_rows, 1)
    if tile not in EXPERT_TC_TILES:
        raise KernelError(f"expert_rows_tc: a row tile of {tile}")
    max_tiles = (plan.numel() - 1) // 3 if plan is not None else 0
    _check(_lib().af_expert_rows_tc(_ptr(out), _ptr(a), _ptr(w0), _ptr(w1, allow_none=True), c_int(E),
                                    _ptr(perm, "perm", torch.int32, allow_none=True),
                                    _ptr(plan, "plan", torch.int32, allow_none=True),
                                    _ptr(pair_weight, "pair_weight", torch.float32, allow_none=True),
                                    _ptr(scale_out, "scale_out", torch.float32, allow_none=True), c_int(n_rows),
                                    c_int(n_tokens), c_int(top), c_int(max_tiles), c_int(tile), c_int(N), c_int(K),
                                    c_float(limit), c_int(EXPERT_ACTS[act]),
                                    _ptr(error_word(a.device), "err", torch.int32), _stream()))


# ---------------------------------------------------------------- a residual stream in several copies

HC_MAX_STREAMS = 16


def _hc_stream(x, S: int, W: int, who: str):
    if x.dtype != torch.float32 or x.dim() != 2 or x.shape[1] != S * W or not x.is_contiguous():
        raise KernelError(f"{who}: the streams are contiguous float32 [tokens, {S} * {W}]")
    if not 1 <= S <= HC_MAX_STREAMS:
        raise KernelError(f"{who}: 1 to {HC_MAX_STREAMS} streams")


def hc_read(y, x, in_w, w, eps: float, offset: float, S: int) -> None:
    """y = norm(sum_s in_w[s] x[:, s]) * (offset + w): x float32 [T, S * W] (stream after stream), y [T, W]."""
    T, W = y.shape
    _hc_stream(x, S, W, "hc_read")
    if in_w.numel() != S or w.numel() != W or not y.is_contiguous():
        raise KernelError("hc_read: one factor a stream, a weight of the row's size")
    _check(_lib().af_hc_read(_ptr(y), c_int(dtype_code(y.dtype)), _ptr(x), _ptr(in_w, "in_w", torch.float32),
                             _ptr(w, "w", torch.float32), c_float(eps), c_float(offset), c_int(T), c_int(S), c_int(W),
                             _stream()))


def hc_write(x, terms, mix, out_w, S: int, scale=None, y=None, in_next=None, w_next=None, eps: float = 0.0,
             offset: float = 0.0) -> None:
    """Every stream from the old ones and a sublayer's result r = sum of the ``terms`` (as in
    :func:`add_scaled_rmsnorm`; one or two), times the per-channel ``scale`` when given:
    x[:, t] <- sum_s mix[s, t] x[:, s] + out_w[t] r.  With ``y``: also y = norm(sum_s in_next[s] x[:, s]) *
    (offset + w_next) of the new streams.  x float32 [T, S * W]; mix float32 [S, S]."""
    T = x.shape[0]
    W = x.shape[1] // S
    _hc_stream(x, S, W, "hc_write")
    if not 1 <= len(terms) <= 2:
        raise KernelError("hc_write: one or two terms")
    if mix.numel() != S * S or out_w.numel() != S or not mix.is_contiguous() or (scale is not None and scale.numel() != W):
        raise KernelError("hc_write: mix [S, S], out_w [S], scale [W]")
    if y is not None and (tuple(y.shape) != (T, W) or not y.is_contiguous() or in_next is None or in_next.numel() != S
                          or w_next is None or w_next.numel() != W):
        raise KernelError("hc_write: the next read wants y [T, W], in_next [S] and w_next [W]")
    a, sa = terms[0]
    b, sb = terms[1] if len(terms) > 1 else (None, 0.0)
    barg = _term_arg(b, T, W, "hc_write") if b is not None else (ctypes.c_void_p(0), c_int(F32), c_int(1))
    _check(_lib().af_hc_write(
        _ptr(x), *_term_arg(a, T, W, "hc_write"), c_float(sa), *barg, c_float(sb),
        _ptr(scale, "scale", torch.float32, allow_none=True), _ptr(mix, "mix", torch.float32),
        _ptr(out_w, "out_w", torch.float32), _ptr(in_next, "in_next", torch.float32, allow_none=True),
        _ptr(w_next, "w_next", torch.float32, allow_none=True), c_float(eps), c_float(offset),
        _ptr(y, "y", allow_none=True), c_int(dtype_code(y.dtype) if y is not None else F32), c_int(T), c_int(S), c_int(W),
        _stream()))


def stream_copy(x, e, S: int) -> None:
    """x[:, s] = e for every stream s: e float32 [T, W], x float32 [T, S * W]."""
    T, W = e.shape
    _hc_stream(x, S, W, "stream_copy")
    if e.dtype != torch.float32 or not e.is_contiguous() or x.shape[0] != T:
        raise KernelError("stream_copy: e contiguous float32 [T, W]")
    _check(_lib().af_stream_copy(_ptr(x), _ptr(e), c_int(T), c_int(S), c_int(W), _stream()))


def stream_sum(out, x, S: int) -> None:
    """out = sum_s x[:, s] (32-bit, in index order)."""
    T, W = out.shape
    _hc_stream(x, S, W, "stream_sum")
    if out.dtype != torch.float32 or not out.is_contiguous() or x.shape[0] != T:
        raise KernelError("stream_sum: out contiguous float32 [T, W]")
    _check(_lib().af_stream_sum(_ptr(out), _ptr(x), c_int(T), c_int(S), c_int(W), _stream()))


# ---------------------------------------------------------------- gated linear attention, differential attention

def channel_decay(alpha, proj, off_low: int, w2t, bias, tau: float) -> None:
    """alpha [T, n] float32 = sigmoid(bias + low w2t)^(1 / tau), ``low`` the ``rank`` columns of the packed float32
    projection rows at ``off_low``, w2t float32 [rank, n]."""
    T, n = alpha.shape
    rank = w2t.shape[0]
    if alpha.dtype != torch.float32 or not alpha.is_contiguous() or tuple(w2t.shape) != (rank, n) or not w2t.is_contiguous() \
            or bias.numel() != n or off_low + rank > proj.shape[1] or proj.shape[0] != T:
        raise KernelError("channel_decay: alpha float32 [T, n], w2t [rank, n], bias [n], the low-rank section inside the row")
    pp, ld = _f32_rows(proj, "proj")
    _check(_lib().af_channel_decay(_ptr(alpha), pp, ld, c_int(off_low), _ptr(w2t, "w2t", torch.float32),
                                   _ptr(bias, "bias", torch.float32), c_int(rank), c_int(T), c_int(n), c_float(tau),
                                   _stream()))


SCAN_CHUNK = 128     # tokens of a chunk when a long prompt's scan is cut into chunks that run side by side


class _ChunkBatch:
    """What ``state_scan`` reads of a batch, with the chunks of a step standing for its sequences."""

    def __init__(self, seq_starts, slots, n_seqs):
        self.seq_starts, self.slots, self.n_seqs = seq_starts, slots, n_seqs


def _scan_chunks(batch, chunk: int):
    """The chunks of a prefill step's sequences (made on the host once a step, kept in ``batch.aux``): device
    tensors chunk_starts [n_chunks + 1], seq_first_chunk [n_seqs + 1], tiles [n_tiles, 3] = (first row, rows <= 32,
    chunk), the chunks' own slots 0 .. n_chunks - 1, and the counts."""
    key = ("scan_chunks", chunk)
    if key not in batch.aux:
        starts, first, tiles, row = [], [0], [], 0
        for n in batch.seq_lens:
            for c0 in range(0, n, chunk):
                rows = min(chunk, n - c0)
                for t0 in range(0, rows, 32):
                    tiles.append((row + c0 + t0, min(32, rows - t0), len(starts)))
                starts.append(row + c0)
            row += n
            first.append(len(starts))
        starts.append(row)
        n_chunks = len(starts) - 1
        flat = starts + first + [x for t in tiles for x in t] + list(range(n_chunks))
        dev = torch.tensor(flat, dtype=torch.int32).to(batch.tokens.device)
        a, b, c = len(starts), len(starts) + len(first), len(starts) + len(first) + 3 * len(tiles)
        batch.aux[key] = (dev[:a], dev[a:b], dev[b:c], dev[c:], n_chunks, len(tiles))
    return batch.aux[key]


def state_scan_chunked(out, r, k, v, w, state, batch, heads: int, dk: int, dv: int, chunk: int = SCAN_CHUNK) -> None:
    """:func:`state_scan` with the rule ``channel`` for a prefill step of few, long sequences: every sequence is cut
    into chunks of ``chunk`` tokens that are scanned side by side from zero states, then joined (the decays
    cumulated within a chunk, the states carried from chunk to chunk, every token's output corrected by what its
    chunk's entering state adds): the same sums in another order, all in 32 bits."""
    T = out.shape[0]
    if tuple(w.shape) != (T, heads * dk):
        raise KernelError(f"state_scan_chunked: a decay per key channel and token, [{T}, {heads * dk}]")
    chunk_starts, seq_first, tiles, own_slots, n_chunks, n_tiles = _scan_chunks(batch, chunk)
    local = torch.zeros(n_chunks, heads, dv, dk, dtype=torch.float32, device=out.device)
    state_scan("channel", out, r, k, v, local, _ChunkBatch(chunk_starts, own_slots, n_chunks), heads, dk, dv, w=w)
    A = torch.empty(T, heads * dk, dtype=torch.float32, device=out.device)
    op, ots = _f32_rows(out, "out")
    rp, rts = _f32_rows(r, "r")
    wp, wts = _f32_rows(w, "w")
    i32 = torch.int32
    _check(_lib().af_chunk_join(op, ots, rp, rts, wp, wts, _ptr(A), _ptr(local), _ptr(state, "state", torch.float32),
                                _ptr(chunk_starts, "chunk_starts", i32), _ptr(seq_first, "seq_first", i32),
                                _ptr(tiles, "tiles", i32), _ptr(batch.slots, "slots", i32), c_int(n_chunks),
                                c_int(batch.n_seqs), c_int(n_tiles), c_int(heads), c_int(dk), c_int(dv), _stream()))


def conv_pack(qkv, proj, batch, H: int, G: int, d: int, dv: int, pk: int, pv: int, bias=None, taps_w=None, history=None,
              temp_coef: float = 0.0, temp_every: int = 0, kv=None) -> None:
    """From float32 projection rows [q (H heads of two maps of d) | k (G heads of two maps) | v (G heads of dv)], plus
    ``bias``: a causal convolution over time on every channel (``taps_w`` float32 [taps, channels], the last tap on
    the token itself; inputs before the step come from ``history`` float32 [slots, taps - 1, channels], which is
    left holding the sequence's last taps - 1 inputs), the query temperature 1 + temp_coef ln(floor((p + 1) /
    temp_every) + 1), and the packing for the grouped attention kernels with every map a head of its own:
    ``qkv`` [T, (2 H + 2 G) pk + 2 G pv] of the compute dtype = 2 H query heads (group by group, first map's heads
    then second map's), 2 G key heads (group, map), 2 G value heads (a group's values twice); heads ``pk`` / ``pv``
    elements apart, zeros behind their own.  With ``kv`` the k and v heads also go to each token's cache row."""
    T = proj.shape[0]
    C = H * 2 * d + G * 2 * d + G * dv
    taps = 1 if taps_w is None else taps_w.shape[0]
    if proj.shape[1] < C or tuple(qkv.shape) != (T, (2 * H + 2 * G) * pk + 2 * G * pv) or pk < d or pv < dv or H % G:
        raise KernelError("conv_pack: shapes of the projection and the packed rows do not fit")
    if taps_w is not None and (tuple(taps_w.shape) != (taps, C) or taps_w.dtype != torch.float32 or not taps_w.is_contiguous()):
        raise KernelError(f"conv_pack: taps float32 [taps, {C}]")
    if taps > 1 and (history is None or history.dtype != torch.float32 or tuple(history.shape[1:]) != (taps - 1, C)
                     or not history.is_contiguous()):
        raise KernelError(f"conv_pack: a history float32 [slots, {taps - 1}, {C}]")
    if bias is not None and bias.numel() != C:
        raise KernelError(f"conv_pack: a bias of {C} values")
    kc = vc = pt = None
    max_pages = ring = 0
    if kv is not None:
        kc, vc, pt, ring = kv.k, kv.v, kv.page_table, kv.ring_rows
        if kc.dtype != qkv.dtype or tuple(kc.shape[1:]) != (2 * G, PAGE, pk) or vc is None \
                or tuple(vc.shape[1:]) != (2 * G, PAGE, pv) or not kc.is_contiguous() or not vc.is_contiguous():
            raise KernelError(f"conv_pack: cache pages must be [pages, {2 * G}, {PAGE}, {pk}] (values {pv}) of the rows' dtype")
        max_pages = pt.shape[1]
    pp, ld = _f32_rows(proj, "proj")
    i32 = torch.int32
    _check(_lib().af_conv_pack(
        _ptr(qkv), c_int(dtype_code(qkv.dtype)), c_longlong(_rows(qkv, "qkv")), pp, ld,
        _ptr(bias, "bias", torch.float32, allow_none=True), _ptr(taps_w, "taps_w", torch.float32, allow_none=True),
        _ptr(history if taps > 1 else None, "history", torch.float32, allow_none=True),
        _ptr(batch.positions, "positions", i32), _ptr(batch.seq_of_token, "seq_of_token", i32),
        _ptr(batch.slots, "slots", i32), _ptr(batch.len_after, "len_after", i32), _ptr(batch.seq_starts, "seq_starts", i32),
        c_int(T), c_int(batch.n_seqs), c_int(taps), c_int(H), c_int(G), c_int(d), c_int(dv), c_int(pk), c_int(pv),
        c_float(temp_coef), c_int(temp_every), _ptr(kc, allow_none=True), _ptr(vc, allow_none=True),
        _ptr(pt, "page_table", i32, allow_none=True), c_int(max_pages), c_int(ring), _stream()))


def diff_join(y, ctx, gate, H: int, G: int, dv: int, pv: int, lam: float, eps: float, post: float, ones: int = 0) -> None:
    """Per token and head h: o = a1 - lam a2 with a1, a2 the outputs of the head's two maps in ``ctx`` [T, 2 H pv]
    (ordered as :func:`conv_pack` orders the queries), o / sqrt(mean(o^2) + eps) * post * sigmoid(gate[t, h]),
    into y [T, >= H dv + ones]: the heads side by side, then ``ones`` columns of 1, then zeros.  ``gate``: float32
    rows [T, H dv] (a column section is fine) or None."""
    T = ctx.shape[0]
    if tuple(ctx.shape) != (T, 2 * H * pv) or y.shape[0] != T or y.shape[1] < H * dv + ones or y.dtype != ctx.dtype:
        raise KernelError("diff_join: shapes or dtypes do not fit")
    gp, gts = _f32_rows(gate, "gate") if gate is not None else (ctypes.c_void_p(0), c_longlong(0))
    _check(_lib().af_diff_join(_ptr(y), c_longlong(_rows(y, "y")), _ptr(ctx), c_longlong(_rows(ctx, "ctx")),
                               c_int(dtype_code(ctx.dtype)), gp, gts, c_int(T), c_int(H), c_int(G), c_int(dv), c_int(pv),
                               c_float(lam), c_float(eps), c_float(post), c_int(ones), _stream()))


__all__ = [n for n in dir() if not n.startswith("_")]
