"""Python face of the CUDA kernels: torch tensors in, a launch on the current stream out.

There is no CPU or library fallback here: every function launches a kernel of ``csrc/``
and raises :class:`KernelError` if the library is missing, the tensors are not on a CUDA
device, or a size is outside what the kernel takes.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from . import build


class KernelError(RuntimeError):
    pass


F32, BF16 = 0, 1
_DT = {torch.float32: F32, torch.bfloat16: BF16}


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DT[dtype]
    except KeyError:
        raise KernelError(f"kernels take float32 and bfloat16, not {dtype}") from None


def _ptr(t: torch.Tensor | None):
    if t is None:
        return c_void_p(0)
    if not t.is_cuda:
        raise KernelError(
            "a tensor on the CPU reached a CUDA kernel: this engine has no CPU path"
        )
    return c_void_p(t.data_ptr())


_scoped_stream = None


def _stream():
    if _scoped_stream is not None:
        return _scoped_stream
    return c_void_p(torch.cuda.current_stream().cuda_stream)


class stream_scope:
    """Looks the current CUDA stream up once for every launch made inside the ``with`` block (the
    look-up costs a third of a launch's host time).  The stream must not be switched inside."""

    def __enter__(self):
        global _scoped_stream
        self.prev = _scoped_stream
        _scoped_stream = c_void_p(torch.cuda.current_stream().cuda_stream)
        return self

    def __exit__(self, *exc):
        global _scoped_stream
        _scoped_stream = self.prev


launches = 0   # kernels launched through this module (a captured graph counts its launches once)


def _check(lib, code: int, what: str):
    global launches
    launches += 1
    if code != 0:
        raise KernelError(f"{what}: {lib.mhb_last_error().decode()}")


def _contig(t: torch.Tensor, name: str):
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")


# ---------------------------------------------------------------------------------------
def embed(table, tokens, out, status=None):
    """out[t] = table[tokens[t]] as float32; ids outside the table give zeros and set status bit 0."""
    lib = build.load("elementwise")
    T, H = out.shape
    _check(lib, lib.mhb_embed(_ptr(table), c_int(dtype_code(table.dtype)), _ptr(tokens), _ptr(out),
                              c_int(T), c_int(H), c_int(table.shape[0]), _ptr(status), _stream()),
           "embed")


def add_rmsnorm(x, weight, eps, out, delta=None, nsplit=1, split_stride=0, rows=None):
    """out[r] = rmsnorm(x[s] + delta[s]) * weight with s = rows[r] if rows is given else r.

    Without ``rows`` and with ``delta`` the sum is written back to ``x`` (the residual).
    ``delta`` may be ``nsplit`` float32 partial matrices ``split_stride`` elements apart.
    """
    lib = build.load("elementwise")
    R, H = out.shape
    ddt = dtype_code(delta.dtype) if delta is not None else F32
    _check(lib, lib.mhb_add_rmsnorm(_ptr(x), _ptr(delta), c_int(ddt), c_int(nsplit),
                                    c_longlong(split_stride), _ptr(weight), c_float(eps),
                                    _ptr(rows), _ptr(out), c_int(dtype_code(out.dtype)),
                                    c_int(R), c_int(H), _stream()), "add_rmsnorm")


def residual_add(x, delta, nsplit=1, split_stride=0):
    lib = build.load("elementwise")
    _check(lib, lib.mhb_residual_add(_ptr(x), _ptr(delta), c_int(dtype_code(delta.dtype)),
                                     c_int(nsplit), c_longlong(split_stride),
                                     c_longlong(x.numel()), _stream()), "residual_add")


def rope_append(qkv, bias, positions, tok_seg, block_table, inv_freq, q_out, cache, *, nq, nkv, d,
                page_size, write_kv=True, rotary_dim=None, interleaved=False, nsplit=1, split_stride=0,
                status=None):
    """Bias + rotary encoding of q and k, q to ``q_out``, k and v into the cache pages.

    ``cache`` is one layer's pool [pages, 2, nkv, page_size, d]; ``block_table`` [S, width]
    holds the page ids of each segment of the batch, ``tok_seg`` [T] the segment of a token.
    ``rotary_dim``: how many leading elements of a head are rotated (None: all of them when
    ``inv_freq`` is given, else none); ``interleaved``: pairs (2i, 2i+1) instead of (i, i + rotary_dim/2).
    """
    lib = build.load("elementwise")
    T = q_out.shape[0]
    if cache.dtype != q_out.dtype:
        raise KernelError("rope_append: cache and activations must have one dtype")
    if rotary_dim is None:
        rotary_dim = d if inv_freq is not None else 0
    if rotary_dim and (inv_freq is None or inv_freq.numel() != rotary_dim // 2):
        raise KernelError(f"rope_append: {rotary_dim} rotated elements need {rotary_dim // 2} frequencies")
    _check(lib, lib.mhb_rope_append(
        _ptr(qkv), c_int(dtype_code(qkv.dtype)), c_int(nsplit), c_longlong(split_stride),
        _ptr(bias), _ptr(positions), _ptr(tok_seg), _ptr(block_table),
        c_int(block_table.shape[-1]), _ptr(inv_freq), _ptr(q_out), _ptr(cache),
        c_int(dtype_code(q_out.dtype)), c_int(T), c_int(nq), c_int(nkv), c_int(d),
        c_int(page_size), c_int(cache.shape[0]), c_int(1 if write_kv else 0),
        c_int(rotary_dim), c_int(1 if interleaved else 0), _ptr(status), _stream()), "rope_append")


def swiglu(gate_up, out, nsplit=1, split_stride=0, block=None):
    """out[t, i] = silu(gate_i) * up_i; gate_up[t] holds blocks of ``block`` gate values followed by
    the up values of the same indices (default: one block, [gate | up])."""
    lib = build.load("elementwise")
    T, I = out.shape
    _check(lib, lib.mhb_swiglu(_ptr(gate_up), c_int(dtype_code(gate_up.dtype)), c_int(nsplit),
                               c_longlong(split_stride), _ptr(out), c_int(dtype_code(out.dtype)),
                               c_int(T), c_int(I), c_int(block or I), _stream()), "swiglu")


def gemm_simt(a, w, out, bias=None, nsplit=1, split_stride=0):
    """out[M, N] = a[M, K] @ w[N, K]^T (+ bias) with float32 accumulation on the CUDA cores."""
    lib = build.load("gemm_simt")
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise KernelError(f"gemm: a is [{M},{K}] but w is {list(w.shape)}")
    if a.stride(1) != 1 or w.stride(1) != 1 or out.stride(-1) != 1:
        raise KernelError("gemm: the last dimension must be contiguous")
    _check(lib, lib.mhb_gemm_simt(
        _ptr(a), c_int(dtype_code(a.dtype)), _ptr(w), c_int(dtype_code(w.dtype)), _ptr(out),
        c_int(dtype_code(out.dtype)), _ptr(bias), c_int(M), c_int(N), c_int(K),
        c_longlong(a.stride(0)), c_longlong(w.stride(0)), c_longlong(out.stride(-2)),
        c_int(nsplit), c_longlong(split_stride), _stream()), "gemm_simt")


STREAM_K_PARTIAL_FLOATS = 2 * 160 * 128 * 256     # workspace of the persistent product: two tiles per CTA
STREAM_K_FLAGS = 4 << 16                            # a counter for each quarter of each tile


def stream_k_scratch(device):
    """(partials, flags) for the persistent product: CTAs that share a tile's K range exchange
    float32 partial tiles through ``partials`` and count in ``flags`` (zero before and after)."""
    return (torch.empty(STREAM_K_PARTIAL_FLOATS, dtype=torch.float32, device=device),
            torch.zeros(STREAM_K_FLAGS, dtype=torch.int32, device=device))


def _scratch_ptrs(scratch):
    if scratch is None:
        return c_void_p(None), c_void_p(None)
    partials, flags = scratch
    if partials.numel() < STREAM_K_PARTIAL_FLOATS or flags.numel() < STREAM_K_FLAGS:
        raise KernelError("gemm_tc: the stream-K scratch is too small")
    return _ptr(partials), _ptr(flags)


class gemm_tc_wait_limit:
    """Inside the block the bounded waits of the persistent product give up after ``limit`` iterations
    instead of about a million: for tests that make a wait run out on purpose (a flag that nothing
    sets) and check that the kernel reports it (status bit 4) and leaves in order."""

    def __init__(self, limit: int):
        self.limit = limit

    def __enter__(self):
        lib = build.load("gemm_tc")
        lib.mhb_gemm_tc_wait_limit.restype = ctypes.c_uint
        self.before = lib.mhb_gemm_tc_wait_limit(ctypes.c_uint(self.limit))
        return self

    def __exit__(self, *exc):
        build.load("gemm_tc").mhb_gemm_tc_wait_limit(ctypes.c_uint(self.before))


def gemm_tc(a, w, out, *, swap: bool, bn: int, nsplit=1, split_stride=0, status=None, scratch=None):
    """out[M, N] = a[M, K] @ w[N, K]^T on the tcgen05 tensor cores (bfloat16 in, float32 accumulate).

    ``swap`` streams the weights through the 128-row operand (for few tokens, M <= bn <= 64);
    ``bn`` is the tile width along the other operand, or 0 for the persistent kernel (more than
    64 tokens), which balances its CTAs over tiles and K with ``scratch`` from stream_k_scratch()."""
    lib = build.load("gemm_tc")
    M, K = a.shape
    N = w.shape[0]
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("gemm_tc: operands must be bfloat16")
    if w.shape[1] != K:
        raise KernelError(f"gemm_tc: a is [{M},{K}] but w is {list(w.shape)}")
    if a.stride(1) != 1 or w.stride(1) != 1 or out.stride(-1) != 1:
        raise KernelError("gemm_tc: the last dimension must be contiguous")
    if swap and M > bn:
        raise KernelError(f"gemm_tc: {M} tokens do not fit the swapped tile of {bn}")
    _check(lib, lib.mhb_gemm_tc(
        _ptr(a), _ptr(w), _ptr(out), c_int(dtype_code(out.dtype)), c_int(M), c_int(N), c_int(K),
        c_longlong(a.stride(0)), c_longlong(w.stride(0)), c_longlong(out.stride(-2)),
        c_int(1 if swap else 0), c_int(bn), c_int(nsplit), c_longlong(split_stride),
        *_scratch_ptrs(scratch), _ptr(status), _stream()), "gemm_tc")


def gemm_tc_swiglu(a, w, out, *, swap: bool, bn: int, status=None, scratch=None):
    """out[M, I] = silu(a Wg^T) * (a Wu^T); ``w`` [2 I, K] holds gate and up rows interleaved in
    blocks of 16 (rows 32j..32j+15 gate, 32j+16..32j+31 up)."""
    lib = build.load("gemm_tc")
    M, K = a.shape
    I = out.shape[1]
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("gemm_tc_swiglu: operands and output must be bfloat16")
    if w.shape != (2 * I, K):
        raise KernelError(f"gemm_tc_swiglu: w is {list(w.shape)}, expected [{2 * I}, {K}]")
    if swap and M > bn:
        raise KernelError(f"gemm_tc: {M} tokens do not fit the swapped tile of {bn}")
    _check(lib, lib.mhb_gemm_tc_swiglu(
        _ptr(a), _ptr(w), _ptr(out), c_int(dtype_code(out.dtype)), c_int(M), c_int(I), c_int(K),
        c_longlong(a.stride(0)), c_longlong(w.stride(0)), c_longlong(out.stride(0)),
        c_int(1 if swap else 0), c_int(bn), *_scratch_ptrs(scratch), _ptr(status), _stream()), "gemm_tc_swiglu")


def rope_table(positions, inv_freq, table):
    """table[t] = cos of token t's rotation angles, then their sin (float32, [T, 2 * angles]), for the
    q/k/v product's rotating epilogue."""
    lib = build.load("elementwise")
    T, rdim = table.shape
    if inv_freq.numel() * 2 != rdim or table.dtype != torch.float32 or not table.is_contiguous():
        raise KernelError("rope_table: the table must be float32 [tokens, 2 * frequencies]")
    _check(lib, lib.mhb_rope_table(_ptr(positions), _ptr(inv_freq), _ptr(table), c_int(T), c_int(rdim), _stream()),
           "rope_table")


def gemm_tc_qkv_rope_supports(d: int, rotary_dim: int, interleaved: bool) -> bool:
    """Head sizes and rotations the q/k/v product's rotating epilogue is built for."""
    return d in (64, 128) and 0 <= rotary_dim <= d and rotary_dim % (16 if interleaved else 32) == 0


def gemm_tc_qkv_rope(x, w, bias, cos_sin, positions, tok_seg, block_table, q_out, cache, *, nq, nkv, d,
                     page_size, rotary_dim=None, interleaved=False, write_kv=True, status=None):
    """The stacked q/k/v product of more than 64 tokens whose epilogue adds the bias, rotates q and k
    (``cos_sin`` from rope_table, None for no rotation) and writes q to ``q_out`` and k, v into the
    pages of ``cache`` (one layer's pool)."""
    lib = build.load("gemm_tc")
    M, K = x.shape
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or q_out.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16:
        raise KernelError("gemm_tc_qkv_rope: operands, q and the cache must be bfloat16")
    if tuple(w.shape) != ((nq + 2 * nkv) * d, K) or not cache.is_contiguous() or not q_out.is_contiguous():
        raise KernelError(f"gemm_tc_qkv_rope: w is {list(w.shape)}, expected [{(nq + 2 * nkv) * d}, {K}]; q and the pool must be contiguous")
    if rotary_dim is None:
        rotary_dim = cos_sin.shape[1] if cos_sin is not None else 0
    if rotary_dim and (cos_sin is None or cos_sin.shape != (M, rotary_dim) or cos_sin.dtype != torch.float32):
        raise KernelError("gemm_tc_qkv_rope: the cos/sin table must be float32 [tokens, rotated elements]")
    _check(lib, lib.mhb_gemm_tc_qkv_rope(
        _ptr(x), _ptr(w), c_int(M), c_int(K), c_longlong(x.stride(0)), c_longlong(w.stride(0)), _ptr(bias),
        _ptr(cos_sin), c_int(rotary_dim), c_int(1 if interleaved else 0), _ptr(positions), _ptr(tok_seg),
        _ptr(block_table), c_int(block_table.shape[-1]), _ptr(q_out),
        _ptr(cache), c_int(nq), c_int(nkv), c_int(d), c_int(page_size), c_int(cache.shape[0]),
        c_int(1 if write_kv else 0), _ptr(status), _stream()), "gemm_tc_qkv_rope")


def attention_simt(q, cache, out, part_acc, part_ml, items, num_items, max_items, positions,
                   block_table, tok_part_row, *, nq, nkv, d, page_size, window=0, scale=None):
    lib = build.load("attention_simt")
    if scale is None:
        scale = float(d) ** -0.5
    _check(lib, lib.mhb_attention_simt(
        _ptr(q), _ptr(cache), _ptr(out), c_int(dtype_code(q.dtype)), _ptr(part_acc), _ptr(part_ml),
        _ptr(items), c_int(num_items), c_int(max_items), _ptr(positions), _ptr(block_table),
        c_int(block_table.shape[-1]), _ptr(tok_part_row), c_int(nq), c_int(nkv), c_int(d),
        c_int(page_size), c_int(cache.shape[0]), c_int(window or 0), c_float(scale), _stream()),
        "attention")


MMA_HEAD_DIMS = (32, 64, 96, 128)   # head sizes the tensor-core attention kernel is built for


def attention_mma(q, cache, out, part_acc, part_ml, items, num_items, rows, positions, block_table,
                  tok_part_row, *, nq, nkv, d, page_size, window=0, scale=None, tok_nsplit=None,
                  counters=None):
    """Tensor-core attention (bfloat16) over ``num_items`` items planned for tiles of ``rows`` rows.

    With ``counters`` (int32, zero, one per (token, KV head, chunk of 16 group heads)) the kernel
    merges the key splits itself and leaves the counters zero; else call attention_combine."""
    lib = build.load("attention_mma")
    if q.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16:
        raise KernelError("attention_mma: q and the cache must be bfloat16")
    if scale is None:
        scale = float(d) ** -0.5
    _check(lib, lib.mhb_attention_mma(
        _ptr(q), _ptr(cache), _ptr(out), _ptr(part_acc), _ptr(part_ml), _ptr(items), c_int(num_items),
        c_int(num_items), c_int(rows), _ptr(positions), _ptr(block_table), c_int(block_table.shape[-1]),
        _ptr(tok_part_row), _ptr(tok_nsplit), _ptr(counters), c_int(nq), c_int(nkv), c_int(d),
        c_int(page_size), c_int(cache.shape[0]), c_int(window or 0), c_float(scale), _stream()),
        "attention_mma")


def attention_tma_supports(d: int, page_size: int) -> bool:
    """Head sizes and page sizes the TMA-fed attention kernel is built for."""
    return d in (64, 128) and 2 <= page_size <= 64 and 64 % page_size == 0


def attention_tma(q, cache, out, part_acc, part_ml, items, num_items, rows, positions, block_table,
                  tok_part_row, *, nq, nkv, d, page_size, window=0, scale=None, tok_nsplit=None,
                  counters=None, status=None, fresh=0):
    """attention_mma with keys and values staged by TMA through a ring of mbarrier-guarded stages.

    ``fresh``: how many positions before an item's first token the kernel launched just before this
    one may have written (the append of the step's own keys); older keys are requested while that
    kernel still runs.  0: it may have written any key."""
    lib = build.load("attention_tma")
    if q.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16:
        raise KernelError("attention_tma: q and the cache must be bfloat16")
    if not cache.is_contiguous():
        raise KernelError("attention_tma: the layer's pool must be contiguous")
    if scale is None:
        scale = float(d) ** -0.5
    _check(lib, lib.mhb_attention_tma(
        _ptr(q), _ptr(cache), _ptr(out), _ptr(part_acc), _ptr(part_ml), _ptr(items), c_int(num_items),
        c_int(num_items), c_int(rows), _ptr(positions), _ptr(block_table), c_int(block_table.shape[-1]),
        _ptr(tok_part_row), _ptr(tok_nsplit), _ptr(counters), c_int(nq), c_int(nkv), c_int(d),
        c_int(page_size), c_int(cache.shape[0]), c_int(window or 0), c_int(fresh), c_float(scale), _ptr(status),
        _stream()), "attention_tma")


DECODE_MAX_SPLITS = 16      # key splits of a token that the fused decode kernel merges in one cluster


def attention_decode_supports(d: int, page_size: int, groups: int, nsplit: int, rotary_dim: int) -> bool:
    """Sizes the fused decode-attention kernel is built for."""
    return (d in (64, 128) and 2 <= page_size <= 64 and 64 % page_size == 0 and 1 <= groups <= 16
            and 1 <= nsplit <= DECODE_MAX_SPLITS and nsplit * -(-groups // nsplit) <= 16
            and 0 <= rotary_dim <= d and rotary_dim % 8 == 0)


_decode_clusters: dict[tuple[int, int], int] = {}


def attention_decode_max_clusters(d: int, nsplit: int) -> int:
    """How many clusters of ``nsplit`` CTAs of the fused decode kernel the device holds at once."""
    key = (d, nsplit)
    if key not in _decode_clusters:
        lib = build.load("attention_decode")
        n = lib.mhb_attention_decode_max_clusters(c_int(d), c_int(nsplit))
        if n < 0:
            raise KernelError(f"attention_decode: {lib.mhb_last_error().decode()}")
        _decode_clusters[key] = n
    return _decode_clusters[key]


def attention_decode(qkv, bias, inv_freq, cache, out, positions, block_table, *, nq, nkv, d, page_size, nsplit,
                     qkv_nsplit=1, qkv_split_stride=0, rotary_dim=None, interleaved=False, window=0, scale=None,
                     status=None, ngroups=1, part_acc=None, part_ml=None):
    """A batch of single new tokens in one kernel: the q/k/v product's float32 partials ``qkv``
    ([qkv_nsplit, T, (nq + 2 nkv) d], ``qkv_split_stride`` elements apart) are summed, biased and
    rotated, k and v are appended to ``cache`` (one layer's pool), every token attends over its
    ``nsplit`` equal shares of keys and the shares are merged inside a thread-block cluster.
    Token i is segment i: ``block_table`` [T, width], ``positions`` [T]; ``out`` [T, nq d] bfloat16.

    ``ngroups`` > 1 cuts every token's keys into ngroups * nsplit shares, ngroups clusters per token and
    KV head: each cluster leaves its part in ``part_acc`` [T * ngroups, nq, d] and ``part_ml``
    [T * ngroups, nq, 2], and ``out`` is written by attention_combine(..., every=ngroups)."""
    lib = build.load("attention_decode")
    T = out.shape[0]
    if qkv.dtype != torch.float32 or cache.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("attention_decode: the product's parts must be float32, cache and output bfloat16")
    if not cache.is_contiguous() or not out.is_contiguous() or qkv.stride(-1) != 1 or qkv.stride(-2) != (nq + 2 * nkv) * d:
        raise KernelError("attention_decode: the pool, the output and the rows of the product must be contiguous")
    if rotary_dim is None:
        rotary_dim = d if inv_freq is not None else 0
    if rotary_dim and (inv_freq is None or inv_freq.numel() != rotary_dim // 2):
        raise KernelError(f"attention_decode: {rotary_dim} rotated elements need {rotary_dim // 2} frequencies")
    if scale is None:
        scale = float(d) ** -0.5
    _check(lib, lib.mhb_attention_decode(
        _ptr(qkv), c_int(qkv_nsplit), c_longlong(qkv_split_stride), _ptr(bias), _ptr(inv_freq), c_int(rotary_dim),
        c_int(1 if interleaved else 0), _ptr(cache), _ptr(out), _ptr(positions), _ptr(block_table),
        c_int(block_table.shape[-1]), c_int(T), c_int(nq), c_int(nkv), c_int(d), c_int(page_size),
        c_int(cache.shape[0]), c_int(window or 0), c_int(nsplit), c_int(ngroups), _ptr(part_acc), _ptr(part_ml),
        c_float(scale), _ptr(status), _stream()),
        "attention_decode")
    if ngroups > 1:
        attention_combine(part_acc, part_ml, None, None, out, nq=nq, d=d, every=ngroups)


def attention_tc(q, cache, out, items, num_items, positions, block_table, *, nq, nkv, d, page_size,
                 window=0, scale=None, status=None, part_acc=None, part_ml=None, tok_part_row=None):
    """tcgen05 attention for long portions: ``items`` planned for tiles of 128 rows; items split
    along the keys write to the partial buffers (then call attention_combine)."""
    lib = build.load("attention_tc")
    if q.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16:
        raise KernelError("attention_tc: q and the cache must be bfloat16")
    if not cache.is_contiguous():
        raise KernelError("attention_tc: the layer's pool must be contiguous")
    if scale is None:
        scale = float(d) ** -0.5
    _check(lib, lib.mhb_attention_tc(
        _ptr(q), _ptr(cache), _ptr(out), _ptr(items), c_int(num_items), _ptr(positions), _ptr(block_table),
        c_int(block_table.shape[-1]), _ptr(tok_part_row), _ptr(part_acc), _ptr(part_ml),
        c_int(nq), c_int(nkv), c_int(d), c_int(page_size),
        c_int(cache.shape[0]), c_int(window or 0), c_float(scale), _ptr(status), _stream()), "attention_tc")


def attention_combine(part_acc, part_ml, tok_part_row, tok_nsplit, out, *, nq, d, every=0):
    """Merge the parts of every token's attention.  ``every`` > 0: each token has exactly that many parts,
    in the rows t * every ... of the partial buffers (the two index arrays may be None)."""
    lib = build.load("attention_simt")
    T = out.shape[0]
    _check(lib, lib.mhb_attention_combine(_ptr(part_acc), _ptr(part_ml), _ptr(tok_part_row),
                                          _ptr(tok_nsplit), _ptr(out), c_int(dtype_code(out.dtype)),
                                          c_int(T), c_int(nq), c_int(d), c_int(every), _stream()),
           "attention_combine")


def sample(logits, temperature, seed, counter, out):
    """out[r] = argmax(logits[r]) where temperature[r] <= 0, else a draw from softmax(logits/T)."""
    lib = build.load("sampling")
    R, V = logits.shape
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise KernelError("sample: logits must be float32 with a contiguous last dimension")
    _check(lib, lib.mhb_sample(_ptr(logits), c_longlong(logits.stride(0)), c_int(R), c_int(V),
                               _ptr(temperature), _ptr(seed), _ptr(counter), _ptr(out), _stream()),
           "sample")
