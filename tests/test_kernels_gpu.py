"""Each CUDA kernel alone against a plain PyTorch float32 reference of the same operation, at
sizes other than the engine's test models (widths and vocabularies that are no power of two,
head sizes in steps of 16, odd group counts)."""
import math

import pytest
import torch

from plain import qwen2_plain as P

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def K():
    from mini_hisparse_b200.kernels import api

    return api


def tol(dtype, scale=1.0):
    if dtype == torch.float32:
        return dict(atol=2e-5 * scale, rtol=2e-5)
    return dict(atol=1.6e-2 * scale, rtol=1.6e-2)


def rnd(*shape, dtype=torch.float32, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


# ---- embedding -----------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
def test_embed(dtype):
    V, H = 777, 200
    table = rnd(V, H, dtype=dtype)
    tokens = torch.tensor([0, 776, 5, 5, 300], dtype=torch.int32, device=DEV)
    out = torch.empty(5, H, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    K().embed(table, tokens, out, status)
    assert torch.equal(out, table.float()[tokens.long()]) and int(status) == 0
    bad = torch.tensor([3, 777, -1], dtype=torch.int32, device=DEV)
    out3 = torch.ones(3, H, device=DEV)
    K().embed(table, bad, out3, status)
    assert int(status) == 1 and torch.equal(out3[1:], torch.zeros(2, H, device=DEV))
    assert torch.equal(out3[0], table.float()[3])


# ---- RMSNorm ------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H", [80, 1000, 3584])
def test_rmsnorm_plain_add_rows_and_splits(dtype, H):
    R, eps = 7, 3e-6
    x = rnd(R, H, seed=1, scale=2.0)
    w = rnd(H, seed=2) * 0.1 + 1
    ref = P.rms_norm(x, w, eps)
    out = torch.empty(R, H, dtype=dtype, device=DEV)
    K().add_rmsnorm(x.clone(), w, eps, out)
    torch.testing.assert_close(out.float(), ref, **tol(dtype, 4))
    # with a delta: the residual is updated in place
    delta = rnd(R, H, dtype=dtype, seed=3)
    xr = x.clone()
    K().add_rmsnorm(xr, w, eps, out, delta=delta)
    torch.testing.assert_close(xr, x + delta.float(), atol=1e-6, rtol=1e-6)
    torch.testing.assert_close(out.float(), P.rms_norm(x + delta.float(), w, eps), **tol(dtype, 4))
    # split partials, summed in order
    parts = rnd(3, R, H, seed=4)
    xr = x.clone()
    K().add_rmsnorm(xr, w, eps, out, delta=parts, nsplit=3, split_stride=parts.stride(0))
    want = x + parts[0] + parts[1] + parts[2]
    torch.testing.assert_close(xr, want, atol=1e-6, rtol=1e-6)
    # selected rows: nothing is written back
    rows = torch.tensor([6, 0, 3], dtype=torch.int32, device=DEV)
    xr = x.clone()
    out3 = torch.empty(3, H, dtype=dtype, device=DEV)
    K().add_rmsnorm(xr, w, eps, out3, delta=delta, rows=rows)
    assert torch.equal(xr, x)
    torch.testing.assert_close(out3.float(), P.rms_norm((x + delta.float())[rows.long()], w, eps), **tol(dtype, 4))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("R,H", [(512, 3584), (1531, 1000), (2048, 72), (700, 4096)])
def test_rmsnorm_many_rows(dtype, R, H):
    """The row-walking kernel of prompt portions (512 rows and more, rows of up to 4,096 elements): more rows
    than CTAs, a last round that not every CTA has, with and without a delta."""
    eps = 1e-5
    x = rnd(R, H, seed=1, scale=2.0)
    x[5] *= 40.0                                # one row far larger than the others: rows do not mix
    w = rnd(H, seed=2) * 0.1 + 1
    delta = rnd(R, H, dtype=dtype, seed=3)
    out = torch.full((R, H), float("nan"), dtype=dtype, device=DEV)
    xr = x.clone()
    K().add_rmsnorm(xr, w, eps, out, delta=delta)
    torch.testing.assert_close(xr, x + delta.float(), atol=1e-6, rtol=1e-6)
    torch.testing.assert_close(out.float(), P.rms_norm(x + delta.float(), w, eps), **tol(dtype, 4))
    out.fill_(float("nan"))
    xr = x.clone()
    K().add_rmsnorm(xr, w, eps, out)
    assert torch.equal(xr, x)
    torch.testing.assert_close(out.float(), P.rms_norm(x, w, eps), **tol(dtype, 4))


def test_residual_add():
    x = rnd(5, 33, seed=1)
    parts = rnd(2, 5, 33, seed=2)
    xr = x.clone()
    K().residual_add(xr, parts, nsplit=2, split_stride=parts.stride(0))
    torch.testing.assert_close(xr, x + parts[0] + parts[1], atol=1e-6, rtol=1e-6)


# ---- matrix product --------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M,N,K_", [(1, 50, 24), (7, 1000, 96), (130, 67, 333), (65, 64, 16), (3, 129, 1)])
def test_gemm_simt(dtype, M, N, K_):
    a = rnd(M, K_, dtype=dtype, seed=1)
    w = rnd(N, K_, dtype=dtype, seed=2)
    bias = rnd(N, seed=3)
    ref = a.float() @ w.float().T
    out = torch.empty(M, N, dtype=torch.float32, device=DEV)
    K().gemm_simt(a, w, out)
    torch.testing.assert_close(out, ref, atol=2e-5 * math.sqrt(K_), rtol=2e-5)
    K().gemm_simt(a, w, out, bias=bias)
    torch.testing.assert_close(out, ref + bias, atol=2e-5 * math.sqrt(K_), rtol=2e-5)
    out_d = torch.empty(M, N, dtype=dtype, device=DEV)
    K().gemm_simt(a, w, out_d)
    torch.testing.assert_close(out_d.float(), ref, **tol(dtype, math.sqrt(K_)))
    parts = torch.full((3, M, N), float("nan"), device=DEV)
    K().gemm_simt(a, w, parts, nsplit=3, split_stride=parts.stride(0))
    torch.testing.assert_close(parts.sum(0), ref, atol=2e-5 * math.sqrt(K_), rtol=2e-5)


def test_gemm_is_true_float32():
    """A product that TF32 or bfloat16 inputs would get wrong by 1e-3 comes out to 1e-6."""
    a = torch.full((4, 64), 1.0 + 2 ** -12, device=DEV)
    w = torch.full((8, 64), 1.0 + 2 ** -12, device=DEV)
    out = torch.empty(4, 8, device=DEV)
    K().gemm_simt(a, w, out)
    exact = 64 * (1.0 + 2 ** -12) ** 2
    assert abs(float(out[0, 0]) - exact) < 1e-4


@pytest.mark.parametrize("M,N,K_,swap,bn,nsplit", [
    (128, 128, 64, False, 128, 1), (200, 300, 136, False, 128, 1), (333, 1000, 3584, False, 256, 1),
    (70, 520, 200, False, 128, 2), (8, 256, 512, True, 16, 1), (1, 777, 96, True, 16, 1),
    (17, 1000, 3584, True, 32, 7), (64, 130, 1024, True, 64, 4), (2048, 2000, 512, False, 256, 1),
])
@pytest.mark.parametrize("out_dtype", DTYPES)
def test_gemm_tensor_core(M, N, K_, swap, bn, nsplit, out_dtype):
    """The tcgen05 product against float32 matmul of the same bfloat16 values: ragged edges in
    every dimension, both operand orders, split K."""
    a = rnd(M, K_, dtype=torch.bfloat16, seed=1)
    w = rnd(N, K_, dtype=torch.bfloat16, seed=2)
    ref = a.float() @ w.float().T
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    if nsplit > 1:
        if out_dtype != torch.float32:
            pytest.skip("partials are float32")
        out = torch.full((nsplit, M, N), float("nan"), device=DEV)
        K().gemm_tc(a, w, out, swap=swap, bn=bn, nsplit=nsplit, split_stride=out.stride(0), status=status)
        got = out.sum(0)
    else:
        out = torch.full((M + 1, N), float("nan"), dtype=out_dtype, device=DEV)
        K().gemm_tc(a, w, out[:M], swap=swap, bn=bn, status=status)
        assert bool(out[M].isnan().all())               # nothing written past the last row
        got = out[:M].float()
    assert int(status) == 0
    if out_dtype == torch.float32:
        torch.testing.assert_close(got, ref, atol=3e-5 * math.sqrt(K_) * 4, rtol=2e-5)
    else:
        torch.testing.assert_close(got, ref, atol=1e-2 * float(ref.abs().max()), rtol=1e-2)


@pytest.mark.parametrize("M,N,K_", [(65, 64, 64), (128, 128, 64), (200, 300, 136), (333, 1000, 3584), (100, 7168, 1024),
                                    (2048, 2000, 512), (1024, 520, 13824), (700, 4608, 3584), (129, 40, 8192),
                                    (2048, 2600, 8192), (1100, 5000, 8256), (2300, 2304, 8960)])
@pytest.mark.parametrize("shared", [True, False])
@pytest.mark.parametrize("out_dtype", DTYPES)
def test_gemm_persistent(M, N, K_, shared, out_dtype):
    """The persistent product: ragged edges, fewer tiles than SMs, and (the last three shapes: a
    long K and a last round that fills a part of the SMs) CTAs that share tiles' K ranges through
    the workspace; the same shapes without a workspace.  Twice in a row: the flags are left zero."""
    a = rnd(M, K_, dtype=torch.bfloat16, seed=1)
    w = rnd(N, K_, dtype=torch.bfloat16, seed=2)
    ref = a.float() @ w.float().T
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    scratch = K().stream_k_scratch(DEV) if shared else None
    outs = []
    for _ in range(2):
        out = torch.full((M + 1, N), float("nan"), dtype=out_dtype, device=DEV)
        K().gemm_tc(a, w, out[:M], swap=False, bn=0, status=status, scratch=scratch)
        assert bool(out[M].isnan().all())
        outs.append(out[:M].float())
    assert int(status) == 0
    if shared:
        assert int(scratch[1].abs().sum()) == 0
    assert torch.equal(outs[0], outs[1])                 # the order of the sums is fixed
    if out_dtype == torch.float32:
        torch.testing.assert_close(outs[0], ref, atol=3e-5 * math.sqrt(K_) * 4, rtol=2e-5)
    else:
        torch.testing.assert_close(outs[0], ref, atol=1e-2 * float(ref.abs().max()), rtol=1e-2)


def test_gemm_persistent_wait_that_runs_out_is_reported_and_the_kernel_stays_usable():
    """A bounded wait made to run out by a flag that nothing sets: the counters through which the CTAs
    that share a tile's K range meet are preset so that their count is never reached.  With a short
    limit the CTAs give up within milliseconds: status bit 4 is set, the kernel returns (its MMAs
    drained, its copies landed, its tensor memory freed), and after the flags are put back to zero
    (what the runner does after such an error) the same product is right again."""
    M, N, K_ = 2300, 2304, 8960                       # its last round of tiles is shared eight ways along K
    a = rnd(M, K_, dtype=torch.bfloat16, seed=1)
    w = rnd(N, K_, dtype=torch.bfloat16, seed=2)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    scratch = K().stream_k_scratch(DEV)
    out = torch.zeros(M, N, dtype=torch.bfloat16, device=DEV)
    scratch[1].fill_(-1000)
    with K().gemm_tc_wait_limit(2000):
        K().gemm_tc(a, w, out, swap=False, bn=0, status=status, scratch=scratch)
        torch.cuda.synchronize()
    assert int(status) & 4
    from mini_hisparse_b200.engine.step import ModelRunner
    assert "tensor-core matrix product" in ModelRunner.status_message(int(status))
    status.zero_()
    scratch[1].zero_()
    K().gemm_tc(a, w, out, swap=False, bn=0, status=status, scratch=scratch)
    assert int(status) == 0 and int(scratch[1].abs().sum()) == 0
    ref = a.float() @ w.float().T
    torch.testing.assert_close(out.float(), ref, atol=1e-2 * float(ref.abs().max()), rtol=1e-2)


@pytest.mark.parametrize("M,I,K_,swap,bn", [(200, 176, 64, False, 256), (2048, 1184, 512, False, 256),
                                              (200, 176, 64, False, 0), (2048, 1184, 512, False, 0), (130, 2000, 3584, False, 0),
                                              (2048, 1312, 8192, False, 0),
                                              (8, 176, 96, True, 16), (33, 304, 3584, True, 64), (1, 18944, 128, True, 16)])
def test_gemm_tensor_core_swiglu_epilogue(M, I, K_, swap, bn):
    """silu(x Wg^T) * (x Wu^T) written by the product's epilogue from block-interleaved weights."""
    x = rnd(M, K_, dtype=torch.bfloat16, seed=1)
    gate = rnd(I, K_, dtype=torch.bfloat16, seed=2, scale=0.2)
    up = rnd(I, K_, dtype=torch.bfloat16, seed=3, scale=0.2)
    w = torch.stack((gate.view(I // 16, 16, K_), up.view(I // 16, 16, K_)), 1).reshape(2 * I, K_).contiguous()
    out = torch.full((M + 1, I), float("nan"), dtype=torch.bfloat16, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    K().gemm_tc_swiglu(x, w, out[:M], swap=swap, bn=bn, status=status,
                       scratch=K().stream_k_scratch(DEV) if bn == 0 else None)
    g, u = x.float() @ gate.float().T, x.float() @ up.float().T
    ref = g * torch.sigmoid(g) * u
    assert int(status) == 0 and bool(out[M].isnan().all())
    torch.testing.assert_close(out[:M].float(), ref, atol=1e-2 * float(ref.abs().max()), rtol=1.6e-2)
    # the stand-alone gate kernel reads the same interleaved layout
    gu = (x.float() @ w.float().T).to(torch.bfloat16)
    out2 = torch.empty(M, I, dtype=torch.bfloat16, device=DEV)
    K().swiglu(gu, out2, block=16)
    torch.testing.assert_close(out2.float(), ref, atol=2e-2 * float(ref.abs().max()), rtol=2e-2)


def test_gemm_tensor_core_refuses_unaligned_k():
    from mini_hisparse_b200.kernels.api import KernelError

    a = rnd(4, 100, dtype=torch.bfloat16)
    w = rnd(9, 100, dtype=torch.bfloat16)
    with pytest.raises(KernelError, match="multiples of 8"):
        K().gemm_tc(a, w, torch.empty(4, 9, device=DEV), swap=True, bn=16)


@pytest.mark.parametrize("nq,nkv,d,P_,T,Kd", [(28, 4, 128, 16, 300, 3584), (3, 1, 64, 32, 70, 192), (5, 5, 128, 8, 129, 256),
                                               (2, 1, 64, 16, 2100, 64)])
@pytest.mark.parametrize("rdim_of,interleaved", [(lambda d: d, False), (lambda d: 0, False), (lambda d: d, True),
                                                 (lambda d: d // 2, False), (lambda d: d // 4 * 3, True)],
                         ids=["half_split", "none", "interleaved", "partial_half_split", "partial_interleaved"])
def test_gemm_qkv_epilogue_rotates_and_appends(nq, nkv, d, P_, T, Kd, rdim_of, interleaved):
    """The q/k/v product whose epilogue adds the bias, rotates and appends to the paged cache,
    against the product followed by the rotary kernel (which has its own test against the plain
    formulas): two segments, one of which starts inside a page; every rotation style."""
    rdim = rdim_of(d)
    assert K().gemm_tc_qkv_rope_supports(d, rdim, interleaved)
    N = (nq + 2 * nkv) * d
    x = rnd(T, Kd, dtype=torch.bfloat16, seed=1)
    w = rnd(N, Kd, dtype=torch.bfloat16, seed=2, scale=1.0 / math.sqrt(Kd))
    bias = rnd(N, seed=3) * 0.1
    theta = 10000.0
    inv = (theta ** (-torch.arange(0, rdim, 2).float() / rdim)).to(DEV) if rdim else None
    n0 = T // 3
    positions = torch.tensor(list(range(37, 37 + n0)) + list(range(0, T - n0)), dtype=torch.int32, device=DEV)
    tok_seg = torch.tensor([0] * n0 + [1] * (T - n0), dtype=torch.int32, device=DEV)
    pages0, pages1 = -(-(37 + n0) // P_), -(-(T - n0) // P_)
    num_pages = pages0 + pages1 + 3
    perm = torch.randperm(num_pages, generator=torch.Generator().manual_seed(5)).tolist()
    table = torch.full((2, max(pages0, pages1)), -1, dtype=torch.int32)
    table[0, :pages0] = torch.tensor(perm[:pages0])
    table[1, :pages1] = torch.tensor(perm[pages0:pages0 + pages1])
    table = table.to(DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    # reference: float32 product, then the rotary kernel
    qkv = torch.empty(T, N, device=DEV)
    K().gemm_simt(x.float(), w.float(), qkv)
    q_ref = torch.empty(T, nq * d, dtype=torch.bfloat16, device=DEV)
    cache_ref = torch.zeros(num_pages, 2, nkv, P_, d, dtype=torch.bfloat16, device=DEV)
    K().rope_append(qkv, bias, positions, tok_seg, table, inv, q_ref, cache_ref, nq=nq, nkv=nkv, d=d, page_size=P_,
                    rotary_dim=rdim, interleaved=interleaved, status=status)
    cs = None
    if rdim:
        cs = torch.empty(T, rdim, device=DEV)
        K().rope_table(positions, inv, cs)
    q = torch.full((T, nq * d), float("nan"), dtype=torch.bfloat16, device=DEV)
    cache = torch.zeros(num_pages, 2, nkv, P_, d, dtype=torch.bfloat16, device=DEV)
    K().gemm_tc_qkv_rope(x, w, bias, cs, positions, tok_seg, table, q, cache, nq=nq, nkv=nkv, d=d, page_size=P_,
                         rotary_dim=rdim, interleaved=interleaved, status=status)
    assert int(status) == 0
    scale = float(qkv.abs().max())
    torch.testing.assert_close(q.float(), q_ref.float(), atol=1e-2 * scale, rtol=1.6e-2)
    torch.testing.assert_close(cache.float(), cache_ref.float(), atol=1e-2 * scale, rtol=1.6e-2)
    written, written_ref = cache.abs().sum(-1) > 0, cache_ref.abs().sum(-1) > 0          # per (page, plane, head, slot)
    assert bool(written_ref.any()) and bool((written == written_ref).all())            # the same slots were written
    # without write access nothing is appended
    cache2 = torch.zeros_like(cache)
    K().gemm_tc_qkv_rope(x, w, bias, cs, positions, tok_seg, table, q, cache2, nq=nq, nkv=nkv, d=d, page_size=P_,
                         rotary_dim=rdim, interleaved=interleaved, write_kv=False, status=status)
    assert int(cache2.abs().sum()) == 0


# ---- rotary + append -----------------------------------------------------------------------------
def plain_rotation(t, positions, theta, rdim, interleaved):
    """The first rdim elements of every head of t [T, heads, d] turned by angle_i = pos * theta^(-2i/rdim):
    pairs (i, i + rdim/2), or (2i, 2i + 1) if interleaved; the rest of the head passes.  With rdim = d
    and half-split pairs this is the reference's rotation (mini_hisparse/model.py:141-151)."""
    if rdim == 0:
        return t
    inv = theta ** (-torch.arange(0, rdim, 2, device=t.device).float() / rdim)
    ang = positions.float()[:, None] * inv[None, :]
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    out = t.clone()
    if interleaved:
        a, b = t[..., 0:rdim:2], t[..., 1:rdim:2]
        out[..., 0:rdim:2], out[..., 1:rdim:2] = a * cos - b * sin, b * cos + a * sin
    else:
        a, b = t[..., : rdim // 2], t[..., rdim // 2: rdim]
        out[..., : rdim // 2], out[..., rdim // 2: rdim] = a * cos - b * sin, b * cos + a * sin
    return out


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,d,P_,rdim,interleaved", [
    (4, 2, 16, 16, 16, False), (3, 1, 32, 32, 32, False), (10, 2, 48, 16, 48, False), (7, 7, 128, 8, 128, False),
    (3, 1, 32, 24, 32, True), (10, 2, 48, 7, 24, False), (2, 2, 64, 16, 40, True), (5, 1, 80, 16, 6, True),
    (2, 1, 18, 16, 10, False), (4, 4, 64, 16, 0, False)])
def test_rope_append(dtype, nq, nkv, d, P_, rdim, interleaved):
    """Every rotation style against the plain rotation: the reference's (half-split pairs over the
    whole head), interleaved pairs, a rotated part of the head (widths that the vector kernel takes and
    widths that only the scalar kernel takes), and none."""
    theta = 50000.0
    T, pages = 21, 9
    width = (nq + 2 * nkv) * d
    qkv = rnd(T, width, seed=1)
    bias = rnd(width, seed=2) * 0.1
    # two segments: one starts at position 37 (inside a page), one at 0
    positions = torch.tensor(list(range(37, 37 + 13)) + list(range(0, 8)), dtype=torch.int32, device=DEV)
    tok_seg = torch.tensor([0] * 13 + [1] * 8, dtype=torch.int32, device=DEV)
    w_pages = -(-(37 + 13) // P_)
    table = torch.full((2, max(w_pages, 2)), -1, dtype=torch.int32)
    perm = torch.randperm(64, generator=torch.Generator().manual_seed(5)).tolist()
    table[0, :w_pages] = torch.tensor(perm[:w_pages])
    table[1, : -(-8 // P_)] = torch.tensor(perm[w_pages : w_pages + -(-8 // P_)])
    table = table.to(DEV)
    cache = torch.zeros(64, 2, nkv, P_, d, dtype=dtype, device=DEV)
    q_out = torch.empty(T, nq * d, dtype=dtype, device=DEV)
    inv = (theta ** (-torch.arange(0, rdim, 2).float() / rdim)).to(DEV) if rdim else None
    K().rope_append(qkv, bias, positions, tok_seg, table, inv, q_out, cache, nq=nq, nkv=nkv, d=d, page_size=P_,
                    rotary_dim=rdim, interleaved=interleaved)
    full = qkv + bias
    q = full[:, : nq * d].view(T, nq, d)
    k = full[:, nq * d : (nq + nkv) * d].view(T, nkv, d)
    v = full[:, (nq + nkv) * d :].view(T, nkv, d)
    if rdim == d and not interleaved:          # the reference's own form, as the plain model computes it
        cos, sin = P.rope_tables(positions, d, theta, torch.float32)
        torch.testing.assert_close(plain_rotation(q, positions, theta, rdim, False), P.rotate(q, cos, sin),
                                   atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(q_out.float().view(T, nq, d), plain_rotation(q, positions, theta, rdim, interleaved),
                               **tol(dtype, 4))
    kr = plain_rotation(k, positions, theta, rdim, interleaved)
    for t in range(T):
        pos, seg = int(positions[t]), int(tok_seg[t])
        page = int(table[seg, pos // P_])
        torch.testing.assert_close(cache[page, 0, :, pos % P_].float(), kr[t], **tol(dtype, 4))
        torch.testing.assert_close(cache[page, 1, :, pos % P_].float(), v[t], **tol(dtype, 4))
    # nothing else was touched
    touched = torch.zeros(64, P_, dtype=torch.bool)
    for t in range(T):
        pos, seg = int(positions[t]), int(tok_seg[t])
        touched[int(table[seg, pos // P_]), pos % P_] = True
    untouched = cache.float().abs().sum((1, 2, 4)).cpu()[~touched]
    assert float(untouched.sum()) == 0.0


def test_rope_append_refuses_a_page_outside_the_pool():
    nq, nkv, d, P_ = 2, 1, 16, 16
    qkv = rnd(1, 4 * d)
    pos = torch.tensor([3], dtype=torch.int32, device=DEV)
    seg = torch.zeros(1, dtype=torch.int32, device=DEV)
    table = torch.tensor([[99]], dtype=torch.int32, device=DEV)
    cache = torch.zeros(4, 2, nkv, P_, d, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    inv = torch.ones(d // 2, device=DEV)
    q_out = torch.empty(1, nq * d, device=DEV)
    K().rope_append(qkv, None, pos, seg, table, inv, q_out, cache, nq=nq, nkv=nkv, d=d, page_size=P_, status=status)
    assert int(status) == 2 and float(cache.abs().sum()) == 0.0


# ---- SwiGLU -------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
def test_swiglu(dtype):
    T, I = 5, 176
    gu = rnd(T, 2 * I, dtype=dtype, seed=1, scale=3)
    out = torch.empty(T, I, dtype=dtype, device=DEV)
    K().swiglu(gu, out)
    g, u = gu.float()[:, :I], gu.float()[:, I:]
    torch.testing.assert_close(out.float(), g * torch.sigmoid(g) * u, **tol(dtype, 8))
    parts = rnd(2, T, 2 * I, seed=2)
    K().swiglu(parts, out, nsplit=2, split_stride=parts.stride(0))
    s = parts.sum(0)
    torch.testing.assert_close(out.float(), s[:, :I] * torch.sigmoid(s[:, :I]) * s[:, I:], **tol(dtype, 8))


# ---- attention -------------------------------------------------------------------------------------
def paged_case(nq, nkv, d, P_, seg_specs, dtype, seed=0):
    """Segments (history, new tokens): K/V of the history AND the new tokens are in shuffled pages
    (the engine appends before it attends)."""
    from mini_hisparse_b200.parts.base import Segment

    pool = sum(-(-(h + n) // P_) for h, n in seg_specs) + 13
    g = torch.Generator().manual_seed(seed)
    perm = torch.randperm(pool, generator=g).tolist()
    cache = torch.zeros(pool, 2, nkv, P_, d, dtype=dtype, device=DEV)
    cache.normal_(generator=torch.Generator(device=DEV).manual_seed(seed))   # stale junk everywhere
    segments, ks, vs, qs, positions = [], [], [], [], []
    width = max(-(-(h + n) // P_) for h, n in seg_specs)
    table = torch.full((len(seg_specs), width), -1, dtype=torch.int32)
    off = 0
    for si, (hist, n) in enumerate(seg_specs):
        total = hist + n
        k = torch.randn(total, nkv, d, generator=g).to(dtype)
        v = torch.randn(total, nkv, d, generator=g).to(dtype)
        q = torch.randn(total, nq, d, generator=g).to(dtype)
        npg = -(-total // P_)
        pages = [perm.pop() for _ in range(npg)]
        table[si, :npg] = torch.tensor(pages)
        for t in range(total):
            cache[pages[t // P_], 0, :, t % P_] = k[t].to(DEV)
            cache[pages[t // P_], 1, :, t % P_] = v[t].to(DEV)
        segments.append(Segment(si, si, hist, n, off))
        ks.append(k), vs.append(v), qs.append(q)
        positions += list(range(hist, total))
        off += n
    return cache, table.to(DEV), segments, qs, ks, vs, torch.tensor(positions, dtype=torch.int32, device=DEV)


def run_attention(nq, nkv, d, P_, seg_specs, dtype, window=None, fixed_nsplit=None, seed=0, edit=None,
                  kernel="simt"):
    from mini_hisparse_b200.parts.attention import ITEM_INTS, AttentionShape, plan_attention

    cache, table, segments, qs, ks, vs, positions = paged_case(nq, nkv, d, P_, seg_specs, dtype, seed)
    if edit:
        edit(qs, ks, vs, cache, table)
    T = sum(n for _, n in seg_specs)
    need = AttentionShape(nq, nkv, window, {"mma": 64, "tc": 128}.get(kernel, 16))
    plan = plan_attention(need, segments, T, 148, fixed_nsplit=fixed_nsplit)
    q = torch.cat([qq[h:] for qq, (h, n) in zip(qs, seg_specs)]).reshape(T, nq * d).to(DEV)
    out = torch.full((T, nq * d), float("nan"), dtype=dtype, device=DEV)
    rows = max(1, plan.part_rows)
    part_acc = torch.full((rows, nq, d), float("nan"), device=DEV)
    part_ml = torch.full((rows, nq, 2), float("nan"), device=DEV)
    items = torch.from_numpy(plan.items).to(DEV).reshape(-1)
    tpr = torch.from_numpy(plan.tok_part_row).to(DEV)
    tns = torch.from_numpy(plan.tok_nsplit).to(DEV)
    n_items = plan.items.shape[0]
    kw = dict(nq=nq, nkv=nkv, d=d, page_size=P_, window=window or 0)
    # "tc": short segments by the TMA-fed mma kernel, long portions by the tcgen05 kernel (the engine's pairing)
    fused = kernel in ("mma", "tc") and seed % 2 == 0     # the kernel merges its own key splits
    if kernel in ("mma", "tc"):
        launch = K().attention_mma if kernel == "mma" else K().attention_tma
        if plan.n_small:
            groups = nq // nkv
            counters = torch.zeros(T * nkv * -(-groups // 16), dtype=torch.int32, device=DEV) if fused else None
            launch(q, cache, out, part_acc, part_ml, items, plan.n_small, 16, positions, table, tpr,
                   tok_nsplit=tns, counters=counters, **kw)
            if fused:
                assert int(counters.abs().sum()) == 0        # left zero for the next launch
        if plan.n_big and kernel == "tc":
            status = torch.zeros(1, dtype=torch.int32, device=DEV)
            K().attention_tc(q, cache, out, items[plan.n_small * ITEM_INTS:], plan.n_big, positions, table,
                             status=status, part_acc=part_acc, part_ml=part_ml, tok_part_row=tpr, **kw)
            assert int(status) == 0
            if plan.big_split:                               # long tiles were split along the keys
                K().attention_combine(part_acc, part_ml, tpr, tns, out, nq=nq, d=d)
        elif plan.n_big:
            launch(q, cache, out, part_acc, part_ml, items[plan.n_small * ITEM_INTS:], plan.n_big, 64,
                   positions, table, tpr, **kw)
    else:
        K().attention_simt(q, cache, out, part_acc, part_ml, items, n_items, n_items, positions, table, tpr, **kw)
    if plan.part_rows and not fused:
        K().attention_combine(part_acc, part_ml, tpr, tns, out, nq=nq, d=d)
    ref = torch.cat([
        P.causal_attention(qq.float(), kk.float(), vv.float(), window=window)[h:]
        for qq, kk, vv, (h, n) in zip(qs, ks, vs, seg_specs)
    ]).reshape(T, nq * d)
    return out.float().cpu(), ref, plan


@pytest.mark.parametrize("nq,nkv,d,P_", [(4, 2, 32, 16), (3, 1, 32, 32), (28, 4, 128, 16), (20, 1, 96, 8),
                                          (6, 3, 64, 7), (40, 2, 128, 16)])
def test_attention_tensor_core_portions_and_decode_mixed(nq, nkv, d, P_):
    """The mma kernel: long portions (64-row tiles), short ones (16-row tiles, warps split the
    keys), portions that start inside a page, and groups larger than a tile."""
    specs = [(0, 137), (45, 19), (130, 1), (63, 2), (200, 70), (0, 1), (5, 16)]
    out, ref, plan = run_attention(nq, nkv, d, P_, specs, torch.bfloat16, kernel="mma")
    assert plan.n_small and plan.n_big
    torch.testing.assert_close(out, ref, **tol(torch.bfloat16, 2))


@pytest.mark.parametrize("nq,nkv,d,P_", [(4, 2, 64, 16), (3, 1, 128, 32), (28, 4, 128, 16), (20, 1, 64, 8),
                                          (6, 3, 128, 64), (256, 2, 128, 16), (40, 2, 128, 4)])
def test_attention_tcgen05_long_portions(nq, nkv, d, P_):
    """The tcgen05 kernel (128-row tiles, S and the O tile in tensor memory) on long portions that
    start at 0 and inside a page, beside short ones that go to the 16-row kernel."""
    specs = [(0, 300), (45, 19), (130, 1), (200, 170), (0, 1), (77, 129)]
    out, ref, plan = run_attention(nq, nkv, d, P_, specs, torch.bfloat16, kernel="tc")
    assert plan.n_small and plan.n_big
    torch.testing.assert_close(out, ref, **tol(torch.bfloat16, 2))


@pytest.mark.parametrize("nq,nkv,d,P_", [(28, 4, 128, 16), (8, 8, 64, 32), (40, 8, 128, 16)])
def test_attention_tcgen05_long_tiles_split_along_the_keys(nq, nkv, d, P_):
    """Portions of some dozens of tokens far into long prompts: fewer 128-row tiles than SMs, so the
    planner splits them along the keys and attention_combine merges the parts; beside them decode
    tokens whose splits the 16-row kernel merges itself."""
    specs = [(3000, 100), (2500, 1), (700, 1), (1800, 40)]
    out, ref, plan = run_attention(nq, nkv, d, P_, specs, torch.bfloat16, kernel="tc")
    assert plan.big_split and plan.n_small
    assert int((plan.items[plan.n_small:, 7] >= 0).sum()) > 0
    torch.testing.assert_close(out, ref, **tol(torch.bfloat16, 2))


@pytest.mark.parametrize("kernel", ["mma", "tc"])
def test_attention_tensor_core_splits_window_and_far_key(kernel):
    bf = torch.bfloat16
    for seed in (0, 1):      # merged inside the kernel, and by attention_combine
        out, ref, plan = run_attention(28, 4, 128, 16, [(700, 1), (33, 1), (1023, 1), (0, 1), (300, 2)], bf,
                                       fixed_nsplit=5, kernel=kernel, seed=seed)
        assert plan.part_rows == 30
        torch.testing.assert_close(out, ref, **tol(bf, 2))
    out, ref, plan = run_attention(40, 2, 64, 16, [(500, 1), (90, 3)], bf, fixed_nsplit=3, kernel=kernel)
    torch.testing.assert_close(out, ref, **tol(bf, 2))          # groups of 20 heads: two chunks per token
    out, ref, plan = run_attention(8, 2, 64, 16, [(2000, 1)], bf, kernel=kernel)
    assert plan.part_rows > 1
    torch.testing.assert_close(out, ref, **tol(bf, 2))
    for window in (1, 5, 16, 40, 64, 65):
        out, ref, _ = run_attention(4, 2, 64, 16, [(0, 150), (77, 3), (100, 1)], bf, window=window, kernel=kernel)
        torch.testing.assert_close(out, ref, **tol(bf, 2))

    def edit(qs, ks, vs, cache, table):
        d = qs[0].shape[-1]
        direction = torch.zeros(d)
        direction[5] = 1.0
        for h in range(qs[0].shape[1]):
            qs[0][-1, h] = direction * 60.0
        ks[0][3, :] = (direction * 8.0).to(ks[0].dtype)
        cache[int(table[0, 0]), 0, :, 3] = ks[0][3].to(cache.device)
    out, ref, _ = run_attention(4, 2, 64, 16, [(640, 1)], bf, edit=edit, kernel=kernel)
    torch.testing.assert_close(out, ref, **tol(bf, 2))
    out2, ref2, _ = run_attention(4, 2, 64, 16, [(0, 641)], bf, edit=edit, kernel=kernel)
    torch.testing.assert_close(out2, ref2, **tol(bf, 2))


@pytest.mark.parametrize("nq,nkv,d,P_,nsplit,qkv_nsplit,rdim,interleaved,window,ngroups", [
    (28, 4, 128, 16, 8, 8, 128, False, None, 1),       # the benchmark's shape: 7 heads per KV head, clusters of 8
    (28, 4, 128, 16, 16, 3, 128, False, None, 1),      # clusters of 16
    (3, 1, 64, 32, 1, 1, 64, False, None, 1),          # one share: nothing to merge
    (32, 2, 128, 8, 4, 2, 64, True, None, 1),          # 16 heads per KV head, interleaved pairs on half the head
    (8, 8, 64, 64, 3, 4, 0, False, None, 1),           # no rotation, one head per KV head, pages of a whole tile
    (12, 4, 128, 4, 6, 1, 96, False, 300, 1),          # a window, tiny pages; 3 heads over 6 shares: some CTAs own no row
    (20, 4, 64, 16, 3, 5, 64, False, None, 1),         # 5 heads over 3 shares: a CTA owns two rows
    (28, 4, 128, 16, 4, 2, 128, False, None, 3),       # three clusters of 4 per token and KV head, merged by attention_combine
    (12, 4, 128, 4, 2, 1, 96, False, 300, 5),          # five clusters of 2, a window: most groups of short histories are empty
    (20, 4, 64, 16, 3, 5, 64, True, None, 2),          # two clusters of 3, a CTA owns two rows
    (3, 1, 64, 32, 1, 1, 64, False, None, 4),          # four clusters of one CTA
])
def test_attention_decode_fused(nq, nkv, d, P_, nsplit, qkv_nsplit, rdim, interleaved, window, ngroups):
    """The decode kernel that does everything between the q/k/v product and the output projection:
    sums the product's parts, adds the bias, rotates, appends k and v to their pages, attends over
    the cache and merges the key shares in its cluster (with several clusters per token and KV head,
    every cluster leaves a part and attention_combine merges them).  Histories of 0, a few, one tile,
    and many keys, some ending at a page's or a tile's edge; one far key among hundreds stands out."""
    check_attention_decode([0, 5, 63, 64, 127, 700, 1023, 333], nq, nkv, d, P_, nsplit, qkv_nsplit, rdim, interleaved,
                           window, ngroups)


def test_attention_decode_fused_more_clusters_than_fit():
    """A batch of 90 tokens with uneven histories and three shares each: 1,080 CTAs in 360 clusters, several
    rounds of them (what the planner chooses for a large batch that would else wait for its longest
    history)."""
    g = torch.Generator().manual_seed(11)
    histories = torch.randint(0, 900, (90,), generator=g).tolist()
    histories[7], histories[50] = 2300, 1999
    check_attention_decode(histories, 28, 4, 128, 16, 3, 2, 128, False, None, 1)


def check_attention_decode(histories, nq, nkv, d, P_, nsplit, qkv_nsplit, rdim, interleaved, window, ngroups):
    bf = torch.bfloat16
    T = len(histories)
    theta = 10000.0
    g = torch.Generator().manual_seed(3)
    width_all = (nq + 2 * nkv) * d
    parts = (torch.randn(qkv_nsplit, T, width_all, generator=g) / math.sqrt(qkv_nsplit)).to(DEV)
    bias = (torch.randn(width_all, generator=g) * 0.1).to(DEV)
    positions = torch.tensor(histories, dtype=torch.int32, device=DEV)
    full = (parts.sum(0) + bias).cpu()
    q = plain_rotation(full[:, : nq * d].view(T, nq, d), positions.cpu(), theta, rdim, interleaved).to(bf).float()
    pages_of = [-(-(h + 1) // P_) for h in histories]
    pool = sum(pages_of) + 5
    perm = torch.randperm(pool, generator=g).tolist()
    cache = torch.randn(pool, 2, nkv, P_, d, generator=g).to(bf).to(DEV)          # stale junk everywhere
    table = torch.full((T, max(pages_of)), -1, dtype=torch.int32)
    ks, vs = [], []
    for i, h in enumerate(histories):
        pages = [perm.pop() for _ in range(pages_of[i])]
        table[i, : len(pages)] = torch.tensor(pages)
        k = torch.randn(h, nkv, d, generator=g).to(bf)
        v = torch.randn(h, nkv, d, generator=g).to(bf)
        if h > 600:          # one far key that the first head of every group looks for: its score stands out
            k[37] = (0.5 * q[i, :: nq // nkv]).to(bf)
        for t in range(h):
            cache[pages[t // P_], 0, :, t % P_] = k[t].to(DEV)
            cache[pages[t // P_], 1, :, t % P_] = v[t].to(DEV)
        ks.append(k), vs.append(v)
    table = table.to(DEV)
    inv = (theta ** (-torch.arange(0, rdim, 2).float() / rdim)).to(DEV) if rdim else None
    before = cache.clone()
    out = torch.full((T, nq * d), float("nan"), dtype=bf, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    assert K().attention_decode_supports(d, P_, nq // nkv, nsplit, rdim)
    extra = {}
    if ngroups > 1:
        extra = dict(ngroups=ngroups, part_acc=torch.full((T * ngroups, nq, d), float("nan"), device=DEV),
                     part_ml=torch.full((T * ngroups, nq, 2), float("nan"), device=DEV))
    K().attention_decode(parts, bias, inv, cache, out, positions, table, nq=nq, nkv=nkv, d=d, page_size=P_,
                         nsplit=nsplit, qkv_nsplit=qkv_nsplit, qkv_split_stride=parts.stride(0), rotary_dim=rdim,
                         interleaved=interleaved, window=window or 0, status=status, **extra)
    assert int(status) == 0
    k_new = plain_rotation(full[:, nq * d: (nq + nkv) * d].view(T, nkv, d), positions.cpu(), theta, rdim, interleaved).to(bf)
    v_new = full[:, (nq + nkv) * d:].view(T, nkv, d).to(bf)
    touched = torch.zeros(pool, P_, dtype=torch.bool)
    for i, h in enumerate(histories):
        k_all = torch.cat((ks[i], k_new[i: i + 1])).float()
        v_all = torch.cat((vs[i], v_new[i: i + 1])).float()
        q_all = torch.zeros(h + 1, nq, d)
        q_all[h] = q[i]
        ref = P.causal_attention(q_all, k_all, v_all, window=window)[h].reshape(-1)
        torch.testing.assert_close(out[i].float().cpu(), ref, **tol(bf, 2))
        page = int(table[i, h // P_])
        torch.testing.assert_close(cache[page, 0, :, h % P_].float().cpu(), k_new[i].float(), **tol(bf, 4))
        torch.testing.assert_close(cache[page, 1, :, h % P_].float().cpu(), v_new[i].float(), **tol(bf, 4))
        touched[page, h % P_] = True
    # nothing but the tokens' own slots was written
    same = (cache == before).all(-1).all(1).all(1).cpu()        # [pool, P]
    assert bool(same[~touched].all())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,d,P_", [(4, 2, 16, 16), (3, 1, 32, 32), (10, 2, 48, 16), (28, 4, 128, 16),
                                          (20, 1, 80, 8), (2, 2, 256, 16), (6, 3, 112, 7)])
def test_attention_prefill_portions_and_decode_mixed(dtype, nq, nkv, d, P_):
    # a whole prompt, a portion at an offset inside a page, a single token, a 2-token portion
    specs = [(0, 37), (45, 19), (130, 1), (63, 2)]
    out, ref, plan = run_attention(nq, nkv, d, P_, specs, dtype)
    torch.testing.assert_close(out, ref, **tol(dtype, 2))


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_split_keys_and_combine(dtype):
    specs = [(700, 1), (33, 1), (1023, 1), (0, 1)]
    out, ref, plan = run_attention(28, 4, 128, 16, specs, dtype, fixed_nsplit=5)
    assert plan.part_rows == 20 and (plan.items[:, 7] >= 0).all()
    torch.testing.assert_close(out, ref, **tol(dtype, 2))
    out, ref, plan = run_attention(8, 2, 64, 16, [(2000, 1)], dtype)      # the planner splits by itself
    assert plan.part_rows > 1
    torch.testing.assert_close(out, ref, **tol(dtype, 2))


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_finds_one_far_key_among_hundreds(dtype):
    """Random keys give near-uniform weights, which would hide a missed page.  Here the query of
    the last token matches key 3 (first page) with a large score: the output must be V[3]."""
    def edit(qs, ks, vs, cache, table):
        d = qs[0].shape[-1]
        direction = torch.zeros(d)
        direction[5] = 1.0
        for h in range(qs[0].shape[1]):
            qs[0][-1, h] = direction * 60.0
        ks[0][3, :] = (direction * 8.0).to(ks[0].dtype)
        page = int(table[0, 0])
        cache[page, 0, :, 3] = ks[0][3].to(cache.device)
    out, ref, _ = run_attention(4, 2, 64, 16, [(640, 1)], dtype, edit=edit)
    torch.testing.assert_close(out, ref, **tol(dtype, 2))
    # and the reference itself is V[3] there, up to the tail of the softmax
    out2, ref2, _ = run_attention(4, 2, 64, 16, [(0, 641)], dtype, edit=edit)
    torch.testing.assert_close(out2[-1], ref2[-1], **tol(dtype, 2))
    torch.testing.assert_close(out[-1], out2[-1], **tol(dtype, 2))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [1, 5, 16, 40])
def test_attention_window_edge(dtype, window):
    """Keys exactly at the window's edge: position - window + 1 is the first key kept."""
    specs = [(0, 50), (77, 3), (100, 1)]
    out, ref, _ = run_attention(4, 2, 32, 16, specs, dtype, window=window)
    torch.testing.assert_close(out, ref, **tol(dtype, 2))


def test_attention_refuses_what_it_cannot_do():
    from mini_hisparse_b200.kernels.api import KernelError
    from mini_hisparse_b200.parts.attention import GQAttention
    from mini_hisparse_b200.parts.spec import PartSpec

    pos = PartSpec.make("rotary", head_dim=40, theta=1e4)
    with pytest.raises(ValueError, match="head_dim 40"):
        GQAttention(PartSpec.make("gq_attention", hidden_size=80, q_heads=2, kv_heads=2, head_dim=40, position=pos))
    with pytest.raises(KernelError, match="CPU"):
        K().embed(torch.zeros(4, 4), torch.zeros(1, dtype=torch.int32), torch.zeros(1, 4))


# ---- sampling -------------------------------------------------------------------------------------
def test_sample_greedy_lowest_index_wins():
    V = 152064 // 8 + 3
    logits = rnd(5, V, seed=3)
    logits[1, 100] = logits[1, 17000] = 50.0
    logits[2, V - 1] = 60.0
    logits[3, 0] = 60.0
    out = torch.empty(5, dtype=torch.int32, device=DEV)
    K().sample(logits, None, None, None, out)
    assert out.tolist() == logits.argmax(-1).tolist()
    assert out[1] == 100 and out[2] == V - 1 and out[3] == 0


def test_sample_temperature_equals_the_plain_draw():
    V, R = 1000, 64
    logits = rnd(R, V, seed=4, scale=2.0)
    temps = torch.tensor([0.8] * (R - 2) + [0.0, 1.5], device=DEV)
    seeds = torch.arange(R, dtype=torch.int64, device=DEV) + 11
    counters = torch.arange(R, dtype=torch.int64, device=DEV) * 3
    out = torch.empty(R, dtype=torch.int32, device=DEV)
    K().sample(logits, temps, seeds, counters, out)
    cpu = logits.cpu()
    for r in range(R):
        if float(temps[r]) == 0:
            assert int(out[r]) == int(cpu[r].argmax())
            continue
        token, margin = P.sample_temperature(cpu[r], float(temps[r]), int(seeds[r]), int(counters[r]))
        assert int(out[r]) == token or margin < 1e-5, (r, int(out[r]), token, margin)
    # the same request draws the same token whatever else is in the batch
    again = torch.empty(3, dtype=torch.int32, device=DEV)
    sel = [5, 40, 9]
    K().sample(logits[sel].contiguous(), temps[sel].contiguous(), seeds[sel].contiguous(),
               counters[sel].contiguous(), again)
    assert again.tolist() == [int(out[i]) for i in sel]
