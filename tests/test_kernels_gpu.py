"""Kernel-level parity tests: every libpk entry point against a plain fp32 PyTorch
restatement of the reference formula (src/ops.cpp of the reference), at the awkward
shape the reference's own kernel tests use (R=67, C=133: tests/test_cuda_ops.cpp:63)
and at aligned shapes that take the vectorised kernels.

Tolerances follow the reference's device tiers (tests/test_cuda_ops.cpp:59-60):
per-element ops 1e-6, row reductions 1e-5 (fp32); bf16 storage adds one rounding of
the result, i.e. a relative 2^-8.
"""
import ctypes
import math

import numpy as np
import pytest
import torch

from tests import pkt
from tests.pkt import BF16, F32, dt, ptr, scratch, stream

pytestmark = pytest.mark.gpu

EW_TOL = 1e-6
ROW_TOL = 1e-5


@pytest.fixture(scope="module")
def pk():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from paperkiln_b200._capi import libpk
    return libpk()


def rnd(*shape, seed=0, lo=-1.5, hi=1.5, dtype=torch.float32):
    g = torch.Generator(device="cpu").manual_seed(seed)
    t = torch.rand(*shape, generator=g) * (hi - lo) + lo
    return t.to(dtype).cuda()


def close(a, b, tol, rel=0.0):
    a, b = a.float(), b.float()
    err = (a - b).abs()
    lim = tol + rel * b.abs()
    assert bool((err <= lim).all()), f"max err {err.max().item():.3e} (limit {tol:.1e} + {rel:.1e}*|ref|)"


def tols(dtype):
    return (EW_TOL, 0.0) if dtype == torch.float32 else (1e-3, 2 ** -7)


SHAPES = [(67, 133), (64, 256), (3, 8)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", SHAPES)
def test_activations(pk, dtype, shape):
    x = rnd(*shape, seed=1, dtype=dtype)
    u = rnd(*shape, seed=2, dtype=dtype)
    dy = rnd(*shape, seed=3, lo=-1, hi=1, dtype=dtype)
    n = x.numel()
    xf, uf, dyf = x.float(), u.float(), dy.float()
    tol, rel = tols(dtype)
    k = 0.7978845608028654

    def run1(fn, a):
        y = torch.empty_like(a)
        pkt.check(fn(stream(), dt(a), ptr(a), ptr(y), n))
        return y

    def run2(fn, a, b):
        y = torch.empty_like(a)
        pkt.check(fn(stream(), dt(a), ptr(a), ptr(b), ptr(y), n))
        return y

    s = torch.sigmoid(xf)
    close(run1(pk.pk_silu_fwd, x), xf / (1 + torch.exp(-xf)), tol, rel)
    close(run2(pk.pk_silu_bwd, dy, x), dyf * s * (1 + xf * (1 - s)), tol * 2, rel)
    close(run1(pk.pk_relu_fwd, x), torch.clamp(xf, min=0), tol, rel)
    close(run2(pk.pk_relu_bwd, dy, x), torch.where(xf > 0, dyf, torch.zeros_like(dyf)), tol, rel)
    inner = k * (xf + 0.044715 * xf ** 3)
    t = torch.tanh(inner)
    close(run1(pk.pk_gelu_fwd, x), xf * 0.5 * (1 + t), tol * 2, rel)
    pdf = 0.5 * (1 - t * t) * k * (1 + 0.134145 * xf * xf)
    close(run2(pk.pk_gelu_bwd, dy, x), dyf * (0.5 * (1 + t) + xf * pdf), tol * 4, rel)
    close(run2(pk.pk_swiglu_fwd, x, u), xf / (1 + torch.exp(-xf)) * uf, tol * 2, rel)
    dg, du = torch.empty_like(x), torch.empty_like(x)
    pkt.check(pk.pk_swiglu_bwd(stream(), dt(x), ptr(dy), ptr(x), ptr(u), ptr(dg), ptr(du), n))
    close(dg, dyf * uf * s * (1 + xf * (1 - s)), tol * 4, rel)
    close(du, dyf * (xf / (1 + torch.exp(-xf))), tol * 2, rel)
    for op, ref in ((0, xf + uf), (1, xf - uf), (2, xf * uf)):
        y = torch.empty_like(x)
        pkt.check(pk.pk_binary(stream(), dt(x), op, ptr(x), ptr(u), ptr(y), n))
        close(y, ref, tol, rel)
    y = torch.empty_like(x)
    pkt.check(pk.pk_scale(stream(), dt(x), ptr(x), 0.37, ptr(y), n))
    close(y, xf * 0.37, tol, rel)


def test_cast_axpy_empty(pk):
    x = rnd(1000, seed=4)
    xb = torch.empty(1000, dtype=torch.bfloat16, device="cuda")
    pkt.check(pk.pk_cast(stream(), F32, ptr(x), BF16, ptr(xb), 1000))
    assert torch.equal(xb, x.to(torch.bfloat16))
    back = torch.empty_like(x)
    pkt.check(pk.pk_cast(stream(), BF16, ptr(xb), F32, ptr(back), 1000))
    assert torch.equal(back, xb.float())
    y = rnd(1000, seed=5)
    y0 = y.clone()
    pkt.check(pk.pk_axpy(stream(), F32, ptr(y), BF16, ptr(xb), 0.5, 1000))
    close(y, y0 + 0.5 * xb.float(), EW_TOL)
    # empty inputs are accepted and do nothing
    pkt.check(pk.pk_axpy(stream(), F32, None, F32, None, 1.0, 0))
    pkt.check(pk.pk_gelu_fwd(stream(), F32, None, None, 0))
    pkt.check(pk.pk_gemm(stream(), F32, F32, 0, 0, 0, 5, 3, None, 3, None, 5, None, 5, 0, None, None, 0))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(67, 133), (40, 128), (300, 768), (33, 2048), (5, 4096 + 8)])
def test_rmsnorm(pk, dtype, shape):
    R, C = shape
    x = rnd(R, C, seed=1, dtype=dtype)
    dy = rnd(R, C, seed=2, lo=-1, hi=1, dtype=dtype)
    w = rnd(C, seed=3, lo=0.5, hi=1.5)
    y = torch.empty_like(x)
    rinv = torch.empty(R, device="cuda")
    pkt.check(pk.pk_rmsnorm_fwd(stream(), dt(x), ptr(x), ptr(w), ptr(y), ptr(rinv), R, C, 1e-5))
    xf, dyf = x.float(), dy.float()
    ri = 1.0 / torch.sqrt((xf * xf).mean(dim=1) + 1e-5)
    tol, rel = (ROW_TOL, 0.0) if dtype == torch.float32 else (1e-3, 2 ** -7)
    close(rinv, ri, ROW_TOL, 1e-5)
    close(y, xf * ri[:, None] * w, tol, rel)
    dx = torch.empty_like(x)
    dw = torch.full((C,), 0.25, device="cuda")  # accumulated into
    sc = scratch(pk.pk_rmsnorm_bwd_scratch_bytes(R, C))
    pkt.check(pk.pk_rmsnorm_bwd(stream(), dt(x), ptr(dy), ptr(x), ptr(w), ptr(rinv), ptr(dx), ptr(dw),
                                ptr(sc), R, C))
    term = (dyf * w * xf).sum(dim=1, keepdim=True)
    dx_ref = ri[:, None] * (dyf * w - xf * (ri * ri)[:, None] * term / C)
    dw_ref = 0.25 + (dyf * xf * ri[:, None]).sum(dim=0)
    close(dx, dx_ref, tol * 4, rel)
    close(dw, dw_ref, 2e-4 if R > 100 else 5e-5, 1e-5)
    # bit-identical when repeated (the recompute contract)
    dx2 = torch.empty_like(x)
    dw2 = torch.full((C,), 0.25, device="cuda")
    pkt.check(pk.pk_rmsnorm_bwd(stream(), dt(x), ptr(dy), ptr(x), ptr(w), ptr(rinv), ptr(dx2), ptr(dw2),
                                ptr(scratch(pk.pk_rmsnorm_bwd_scratch_bytes(R, C))), R, C))
    assert torch.equal(dx, dx2) and torch.equal(dw, dw2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(67, 133), (300, 768), (33, 2048)])
def test_layernorm(pk, dtype, shape):
    R, C = shape
    x = rnd(R, C, seed=1, dtype=dtype)
    dy = rnd(R, C, seed=2, lo=-1, hi=1, dtype=dtype)
    g = rnd(C, seed=3, lo=0.5, hi=1.5)
    b = rnd(C, seed=4, lo=-0.5, hi=0.5)
    y = torch.empty_like(x)
    mean = torch.empty(R, device="cuda")
    rstd = torch.empty(R, device="cuda")
    pkt.check(pk.pk_layernorm_fwd(stream(), dt(x), ptr(x), ptr(g), ptr(b), ptr(y), ptr(mean), ptr(rstd), R, C, 1e-5))
    xf, dyf = x.float(), dy.float()
    mu = xf.mean(dim=1, keepdim=True)
    var = ((xf - mu) ** 2).mean(dim=1, keepdim=True)
    rs = 1.0 / torch.sqrt(var + 1e-5)
    xh = (xf - mu) * rs
    tol, rel = (ROW_TOL, 0.0) if dtype == torch.float32 else (1e-3, 2 ** -7)
    close(y, g * xh + b, tol * 2, rel)
    dx = torch.empty_like(x)
    dg = torch.zeros(C, device="cuda")
    db = torch.zeros(C, device="cuda")
    sc = scratch(pk.pk_layernorm_bwd_scratch_bytes(R, C))
    pkt.check(pk.pk_layernorm_bwd(stream(), dt(x), ptr(dy), ptr(x), ptr(g), ptr(mean), ptr(rstd), ptr(dx),
                                  ptr(dg), ptr(db), ptr(sc), R, C))
    dxh = dyf * g
    m1 = dxh.mean(dim=1, keepdim=True)
    m2 = (dxh * xh).mean(dim=1, keepdim=True)
    close(dx, rs * (dxh - m1 - xh * m2), tol * 8, rel)
    close(dg, (dyf * xh).sum(dim=0), 2e-4, 1e-5)
    close(db, dyf.sum(dim=0), 2e-4, 1e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rope(pk, dtype):
    R, d, hd, nh = 24, 16, 8, 2
    x = rnd(R, 3 * d, seed=6, lo=-1, hi=1, dtype=dtype)
    pos = torch.tensor([i % 12 for i in range(R)], dtype=torch.int32, device="cuda")
    tab = np.zeros((12, hd // 2, 2), dtype=np.float32)
    for p in range(12):
        for j in range(hd // 2):
            inv = np.float32(1.0) / np.float32(np.power(np.float32(10000.0), np.float32(2 * j) / np.float32(hd)))
            th = np.float32(p) * inv
            tab[p, j] = (np.cos(th), np.sin(th))
    tab_d = torch.from_numpy(tab).cuda()
    ref = x.float().clone()
    for col0 in (0, d):
        for h in range(nh):
            for j in range(hd // 2):
                c = col0 + h * hd + 2 * j
                cs = tab_d[pos.long(), j, 0]
                sn = tab_d[pos.long(), j, 1]
                x0, x1 = x.float()[:, c], x.float()[:, c + 1]
                ref[:, c] = x0 * cs - x1 * sn
                ref[:, c + 1] = x0 * sn + x1 * cs
    y = x.clone()
    for col0 in (0, d):
        pkt.check(pk.pk_rope(stream(), dt(y), ptr(y), 3 * d, col0, nh, hd, ptr(pos), ptr(tab_d), 12, R, 0))
    tol, rel = tols(dtype)
    close(y, ref, tol * 2, rel)
    assert torch.equal(y[:, 2 * d:], x[:, 2 * d:])  # v untouched
    # inverse rotation restores the input (fp32: to rounding)
    for col0 in (0, d):
        pkt.check(pk.pk_rope(stream(), dt(y), ptr(y), 3 * d, col0, nh, hd, ptr(pos), ptr(tab_d), 12, R, 1))
    close(y, x, 1e-5 if dtype == torch.float32 else 3e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_bias_colsum_copy_transpose(pk, dtype):
    R, C = 67, 133
    x = rnd(R, C, seed=1, dtype=dtype)
    b = rnd(C, seed=2)
    tol, rel = tols(dtype)
    y = torch.empty_like(x)
    pkt.check(pk.pk_add_bias(stream(), dt(x), ptr(x), ptr(b), ptr(y), R, C))
    close(y, x.float() + b, tol, rel)
    x2 = rnd(64, 256, seed=3, dtype=dtype)
    b2 = rnd(256, seed=4)
    y2 = torch.empty_like(x2)
    pkt.check(pk.pk_add_bias(stream(), dt(x2), ptr(x2), ptr(b2), ptr(y2), 64, 256))
    close(y2, x2.float() + b2, tol, rel)
    out = torch.full((C,), 1.0, device="cuda")
    pkt.check(pk.pk_colsum(stream(), dt(x), ptr(x), ptr(out), ptr(scratch(pk.pk_colsum_scratch_bytes(R, C))), R, C))
    close(out, 1.0 + x.float().sum(dim=0), 5e-5, 1e-5)
    # slice columns 5..38 into a fresh matrix, then scatter-accumulate them back
    sl = torch.empty(R, 33, dtype=dtype, device="cuda")
    pkt.check(pk.pk_copy_cols(stream(), dt(x), ptr(x), C, 5, ptr(sl), 33, 0, R, 33, 0))
    assert torch.equal(sl, x[:, 5:38])
    acc = x.clone()
    pkt.check(pk.pk_copy_cols(stream(), dt(x), ptr(sl), 33, 0, ptr(acc), C, 5, R, 33, 1))
    ref = x.float().clone()
    ref[:, 5:38] += sl.float()
    close(acc, ref, tol, rel)
    # aligned (vector) path
    big = rnd(40, 512, seed=5, dtype=dtype)
    part = torch.empty(40, 128, dtype=dtype, device="cuda")
    pkt.check(pk.pk_copy_cols(stream(), dt(big), ptr(big), 512, 256, ptr(part), 128, 0, 40, 128, 0))
    assert torch.equal(part, big[:, 256:384])
    t = torch.empty(C, R, dtype=dtype, device="cuda")
    pkt.check(pk.pk_transpose(stream(), dt(x), ptr(x), ptr(t), R, C))
    assert torch.equal(t, x.t().contiguous())


@pytest.mark.parametrize("ta,tb", [(False, False), (False, True), (True, False), (True, True)])
def test_gemm_fp32(pk, ta, tb):
    M, N, K = 37, 29, 53  # tests/test_resident_parity.cpp:53-54 shape
    A = rnd(K, M, seed=1, lo=-1, hi=1) if ta else rnd(M, K, seed=1, lo=-1, hi=1)
    B = rnd(N, K, seed=2, lo=-1, hi=1) if tb else rnd(K, N, seed=2, lo=-1, hi=1)
    ref = (A.t() if ta else A).double() @ (B.t() if tb else B).double()
    C = pkt.gemm(A, B, ta=ta, tb=tb)
    assert pk.pk_gemm_last_path() == 0
    close(C, ref.float(), 1e-5)
    bias = rnd(N, seed=3)
    res = rnd(M, N, seed=4)
    C0 = rnd(M, N, seed=5)
    C2 = C0.clone()
    pkt.gemm(A, B, ta=ta, tb=tb, C=C2, accumulate=True, bias=bias, residual=res)
    close(C2, (ref + bias.double() + res.double() + C0.double()).float(), 1e-5)


TC_SHAPES = [(128, 128, 64), (256, 512, 256), (200, 264, 136), (384, 96, 1024), (1000, 2048, 512)]


@pytest.mark.parametrize("ta,tb", [(False, True), (False, False), (True, False), (True, True)])
@pytest.mark.parametrize("mnk", TC_SHAPES)
def test_gemm_bf16_tensor_core(pk, ta, tb, mnk):
    """tcgen05 kernel against fp32 math on the same bf16-rounded inputs, and against the
    SIMT kernel (same inputs, fp32 accumulation in a different order)."""
    M, N, K = mnk
    bf = torch.bfloat16
    A = rnd(K, M, seed=1, lo=-1, hi=1, dtype=bf) if ta else rnd(M, K, seed=1, lo=-1, hi=1, dtype=bf)
    B = rnd(N, K, seed=2, lo=-1, hi=1, dtype=bf) if tb else rnd(K, N, seed=2, lo=-1, hi=1, dtype=bf)
    ref = (A.t() if ta else A).float() @ (B.t() if tb else B).float()
    C = pkt.gemm(A, B, ta=ta, tb=tb, out_dtype=torch.float32)
    assert pk.pk_gemm_last_path() in (2, 3), "tensor-core kernel was not selected"
    st = ctypes.c_int(0)
    pkt.check(pk.pk_gemm_tc_status(ctypes.byref(st), 1))
    assert st.value == 0, "tensor-core kernel reported a wait that gave up"
    atol = 2e-3 * math.sqrt(K / 64)
    close(C, ref, atol, 1e-3)
    pkt.check(pk.pk_gemm_force_simt(1))
    try:
        Cs = pkt.gemm(A, B, ta=ta, tb=tb, out_dtype=torch.float32)
        assert pk.pk_gemm_last_path() == 1
    finally:
        pkt.check(pk.pk_gemm_force_simt(0))
    close(C, Cs, atol, 1e-3)
    # bf16 output with bias + residual, and fp32 accumulate-into (the dW shape)
    bias = rnd(N, seed=3)
    res = rnd(M, N, seed=4, dtype=bf)
    Cb = pkt.gemm(A, B, ta=ta, tb=tb, out_dtype=bf, bias=bias, residual=res)
    close(Cb, ref + bias + res.float(), atol + 2e-2, 2 ** -7)
    C0 = rnd(M, N, seed=5)
    C2 = C0.clone()
    pkt.gemm(A, B, ta=ta, tb=tb, C=C2, accumulate=True)
    close(C2, ref + C0, atol, 1e-3)
    # reproducible bit for bit
    C3 = pkt.gemm(A, B, ta=ta, tb=tb, out_dtype=torch.float32)
    assert torch.equal(C, C3)


@pytest.mark.parametrize("ta,tb", [(False, True), (False, False), (True, False)])
@pytest.mark.parametrize("mnk", [(130, 97, 70), (257, 50257 // 64, 100), (64, 1003, 48)])
def test_gemm_bf16_tensor_core_ragged(pk, ta, tb, mnk):
    """Extents that are not multiples of 8 (a 50257-wide vocabulary) stay on the tensor-core
    kernel as long as the row strides are multiples of 16 bytes."""
    M, N, K = mnk
    bf = torch.bfloat16

    def padded(rows, cols, seed, dtype=bf):
        ld = (cols + 7) // 8 * 8
        buf = torch.full((rows, ld), float("nan"), dtype=dtype, device="cuda")
        buf[:, :cols] = rnd(rows, cols, seed=seed, lo=-1, hi=1, dtype=dtype)
        return buf[:, :cols]

    A = padded(K, M, 1) if ta else padded(M, K, 1)
    B = padded(N, K, 2) if tb else padded(K, N, 2)
    ref = (A.t() if ta else A).float() @ (B.t() if tb else B).float()
    C = padded(M, N, 3, dtype=torch.float32)
    C0 = C.clone()
    pkt.gemm(A, B, ta=ta, tb=tb, C=C, accumulate=True)
    assert pk.pk_gemm_last_path() in (2, 3), "tensor-core kernel was not selected"
    close(C, ref + C0, 2e-3 * math.sqrt(max(K, 64) / 64), 1e-3)
    Cb = padded(M, N, 4)
    pkt.gemm(A, B, ta=ta, tb=tb, C=Cb)
    close(Cb, ref, 3e-2, 2 ** -7)
    st = ctypes.c_int(0)
    pkt.check(pk.pk_gemm_tc_status(ctypes.byref(st), 1))
    assert st.value == 0


@pytest.mark.parametrize("shape", [(4096, 4096, 512), (4096, 2048 + 40, 304), (3000, 4096, 2048)])
@pytest.mark.parametrize("ta,tb", [(False, False), (False, True), (True, False)])
def test_gemm_cta_pair_kernel(pk, shape, ta, tb):
    """The CTA-pair kernel (tcgen05 cta_group::2, 256 x 256 tiles, each CTA loading half of B) gives
    the one-CTA kernel's result bit for bit -- same products, same k order -- for bf16 and fp32
    outputs, with bias / residual / accumulate epilogues and ragged extents."""
    M, N, K = shape
    A = rnd(K, M, seed=1, lo=-1, hi=1, dtype=torch.bfloat16) if ta else rnd(M, K, seed=1, lo=-1, hi=1, dtype=torch.bfloat16)
    B = rnd(N, K, seed=2, lo=-1, hi=1, dtype=torch.bfloat16) if tb else rnd(K, N, seed=2, lo=-1, hi=1, dtype=torch.bfloat16)
    bias = rnd(1, N, seed=3).reshape(N)
    res = rnd(M, N, seed=4, dtype=torch.bfloat16)
    outs = {}
    try:
        for mode in (0, 1):
            pkt.check(pk.pk_gemm_pair_mode(mode))
            Cb = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
            pkt.gemm(A, B, ta=ta, tb=tb, C=Cb, bias=bias, residual=res)
            path = pk.pk_gemm_last_path()
            Cf = torch.ones(M, N, device="cuda")
            pkt.gemm(A, B, ta=ta, tb=tb, C=Cf, accumulate=True)
            outs[mode] = (Cb, Cf, path)
    finally:
        pkt.check(pk.pk_gemm_pair_mode(1))
    st = ctypes.c_int(0)
    pkt.check(pk.pk_gemm_tc_status(ctypes.byref(st), 1))
    assert st.value == 0
    assert outs[0][2] == 2 and outs[1][2] == 3, "the pair kernel was not selected"
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
    ref = (A.t() if ta else A).float() @ (B.t() if tb else B).float()
    close(outs[1][1], ref + 1.0, 2e-3 * math.sqrt(max(K, 64) / 64), 1e-3)


@pytest.mark.parametrize("shape,ta,tb", [((2048, 512, 16384), True, False), ((768, 768, 8192), True, False),
                                         ((300, 200, 8192), False, False), ((896, 16, 8192), True, False),
                                         ((256, 264, 4096 + 64), False, True),
                                         ((2048, 8192, 16384), True, False),   # CTA-pair kernel
                                         ((3072, 896, 16384), False, False)])  # 48 pair tiles: pair kernel because 3 k parts fill it
def test_gemm_split_k(pk, shape, ta, tb):
    """Few output tiles and a long k extent (weight gradients of narrow projections): with a
    workspace the k range is cut into parts whose fp32 partial tiles are added in a fixed order.
    Same result as the unsplit kernel up to the grouping of the sum, reproducible bit for bit,
    with bias / residual / accumulate applied once, ragged extents included."""
    M, N, K = shape
    A = rnd(K, M, seed=1, lo=-1, hi=1, dtype=torch.bfloat16) if ta else rnd(M, K, seed=1, lo=-1, hi=1, dtype=torch.bfloat16)
    B = rnd(N, K, seed=2, lo=-1, hi=1, dtype=torch.bfloat16) if tb else rnd(K, N, seed=2, lo=-1, hi=1, dtype=torch.bfloat16)
    bias = rnd(1, N, seed=3).reshape(N)
    res = rnd(M, N, seed=4, dtype=torch.bfloat16)
    ws = torch.empty(128 << 20, dtype=torch.uint8, device="cuda")
    outs = {}
    try:
        for split in (0, 1, 2):
            pkt.check(pk.pk_gemm_set_workspace(ptr(ws) if split else None, ws.numel() if split else 0))
            Cb = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
            pkt.gemm(A, B, ta=ta, tb=tb, C=Cb, bias=bias, residual=res)
            n1 = pk.pk_gemm_last_splits()
            Cf = torch.ones(M, N, device="cuda")
            pkt.gemm(A, B, ta=ta, tb=tb, C=Cf, accumulate=True)
            outs[split] = (Cb, Cf, n1, pk.pk_gemm_last_splits())
    finally:
        pkt.check(pk.pk_gemm_set_workspace(None, 0))
    st = ctypes.c_int(0)
    pkt.check(pk.pk_gemm_tc_status(ctypes.byref(st), 1))
    assert st.value == 0
    assert outs[0][2] == 1 and outs[0][3] == 1
    assert outs[1][2] > 1 and outs[1][3] > 1, "the k range was not split"
    if shape == (3072, 896, 16384):
        assert pk.pk_gemm_last_path() == 3 and outs[1][2] == 3, "few tiles with a long k loop belong on the pair kernel in three parts"
    assert torch.equal(outs[1][0], outs[2][0]) and torch.equal(outs[1][1], outs[2][1])
    ref = (A.t() if ta else A).float() @ (B.t() if tb else B).float()
    tol = 2e-3 * math.sqrt(max(K, 64) / 64)
    close(outs[1][1], ref + 1.0, tol, 1e-3)
    close(outs[1][1], outs[0][1], tol, 1e-3)
    close(outs[1][0].float(), (ref + bias + res.float()), tol + 0.05, 2 ** -7)


def attn_ref(q, k, v, B, S, Hq, Hkv, dk, scale, causal):
    """fp32 restatement of ops::fused_attention per head (src/ops.cpp:863-934)."""
    q = q.float().view(B, S, Hq, dk).transpose(1, 2)
    k = k.float().view(B, S, Hkv, dk).transpose(1, 2).repeat_interleave(Hq // Hkv, dim=1)
    v = v.float().view(B, S, Hkv, dk).transpose(1, 2).repeat_interleave(Hq // Hkv, dim=1)
    s = (q @ k.transpose(-1, -2)) * scale
    if causal:
        mask = torch.ones(S, S, dtype=torch.bool, device=q.device).tril()
        s = s.masked_fill(~mask, float("-inf"))
    p = torch.softmax(s, dim=-1)
    return (p @ v).transpose(1, 2).reshape(B * S, Hq * dk)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("cfg", [(3, 20, 1, 1, 8, True), (2, 100, 4, 2, 32, True), (2, 67, 2, 2, 64, False),
                                 (1, 130, 2, 1, 128, True), (2, 300, 4, 2, 64, True), (1, 513, 2, 2, 128, True),
                                 (2, 256, 2, 1, 64, False), (1, 1024, 8, 2, 64, True)])
def test_attention(pk, dtype, cfg):
    B, S, Hq, Hkv, dk, causal = cfg
    R = B * S
    q = rnd(R, Hq * dk, seed=1, lo=-1, hi=1, dtype=dtype)
    k = rnd(R, Hkv * dk, seed=2, lo=-1, hi=1, dtype=dtype)
    v = rnd(R, Hkv * dk, seed=3, lo=-1, hi=1, dtype=dtype)
    do = rnd(R, Hq * dk, seed=4, lo=-1, hi=1, dtype=dtype)
    scale = 1.0 / math.sqrt(dk)
    out = torch.empty_like(q)
    lse = torch.empty(R, Hq, device="cuda")
    pkt.check(pk.pk_attn_fwd(stream(), dt(q), ptr(q), Hq * dk, ptr(k), Hkv * dk, ptr(v), Hkv * dk, ptr(out),
                             Hq * dk, ptr(lse), B, S, Hq, Hkv, dk, scale, int(causal)))
    if dtype == torch.bfloat16 and dk in (64, 128):
        assert pk.pk_attn_last_path() == 1, "tensor-core attention was not selected"
        st = ctypes.c_int(0)
        pkt.check(pk.pk_attn_tc_status(ctypes.byref(st), 1))
        assert st.value == 0, "tensor-core attention reported a wait that gave up"
        out2 = torch.empty_like(q)
        lse2 = torch.empty(R, Hq, device="cuda")
        pkt.check(pk.pk_attn_fwd(stream(), dt(q), ptr(q), Hq * dk, ptr(k), Hkv * dk, ptr(v), Hkv * dk, ptr(out2),
                                 Hq * dk, ptr(lse2), B, S, Hq, Hkv, dk, scale, int(causal)))
        assert torch.equal(out, out2) and torch.equal(lse, lse2), "attention forward is not reproducible"
    qf, kf, vf = (t.float().requires_grad_(True) for t in (q, k, v))
    ref = attn_ref(qf, kf, vf, B, S, Hq, Hkv, dk, scale, causal)
    sref = (qf.view(B, S, Hq, dk).transpose(1, 2) @
            kf.view(B, S, Hkv, dk).transpose(1, 2).repeat_interleave(Hq // Hkv, dim=1).transpose(-1, -2)) * scale
    if causal:
        sref = sref.masked_fill(~torch.ones(S, S, dtype=torch.bool, device="cuda").tril(), float("-inf"))
    close(lse, torch.logsumexp(sref, dim=-1).transpose(1, 2).reshape(R, Hq).detach(), 1e-4 if dtype == torch.float32 else 2e-2)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    close(out, ref, tol)
    ref.backward(do.float())
    dq, dkk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    sc = scratch(pk.pk_attn_bwd_scratch_bytes(B, S, Hq))
    pkt.check(pk.pk_attn_bwd(stream(), dt(q), ptr(q), Hq * dk, ptr(k), Hkv * dk, ptr(v), Hkv * dk, ptr(out),
                             Hq * dk, ptr(lse), ptr(do), Hq * dk, ptr(dq), Hq * dk, ptr(dkk), Hkv * dk, ptr(dv),
                             Hkv * dk, ptr(sc), B, S, Hq, Hkv, dk, scale, int(causal)))
    if dtype == torch.bfloat16 and dk in (64, 128):
        assert pk.pk_attn_last_path() == 1, "tensor-core attention backward was not selected"
        st = ctypes.c_int(0)
        pkt.check(pk.pk_attn_tc_status(ctypes.byref(st), 1))
        assert st.value == 0, "tensor-core attention backward reported a wait that gave up"
        dq2, dk2, dv2 = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        pkt.check(pk.pk_attn_bwd(stream(), dt(q), ptr(q), Hq * dk, ptr(k), Hkv * dk, ptr(v), Hkv * dk, ptr(out),
                                 Hq * dk, ptr(lse), ptr(do), Hq * dk, ptr(dq2), Hq * dk, ptr(dk2), Hkv * dk, ptr(dv2),
                                 Hkv * dk, ptr(sc), B, S, Hq, Hkv, dk, scale, int(causal)))
        assert torch.equal(dq, dq2) and torch.equal(dkk, dk2) and torch.equal(dv, dv2), "backward not reproducible"
    gtol = 1e-4 if dtype == torch.float32 else 6e-2
    close(dq, qf.grad, gtol)
    close(dkk, kf.grad, gtol)
    close(dv, vf.grad, gtol)


@pytest.mark.parametrize("cfg", [(2, 200, 2, 1, 64, True), (3, 333, 2, 2, 128, False), (2, 70, 4, 2, 64, True)])
def test_attention_sequences_are_isolated_even_from_infinities(pk, cfg):
    """Exact isolation between stacked sequences (tests/test_batching.cpp:108-120 of the reference)
    when the sequence length is not a multiple of the kernels' tile: the last tile of a sequence
    must not read the next sequence's rows at all. Infinities planted in the LAST sequence's q, k, v
    and upstream gradient must leave every other sequence's outputs and gradients bit-identical
    (a masked score times an infinite value would otherwise give NaN)."""
    B, S, Hq, Hkv, dk, causal = cfg
    R = B * S
    scale = 1.0 / math.sqrt(dk)

    def run(poison):
        q = rnd(R, Hq * dk, seed=21, lo=-1, hi=1, dtype=torch.bfloat16)
        k = rnd(R, Hkv * dk, seed=22, lo=-1, hi=1, dtype=torch.bfloat16)
        v = rnd(R, Hkv * dk, seed=23, lo=-1, hi=1, dtype=torch.bfloat16)
        do = rnd(R, Hq * dk, seed=24, lo=-1, hi=1, dtype=torch.bfloat16)
        if poison:
            for t in (q, k, v, do):
                t[(B - 1) * S:] = float("inf")
        out = torch.empty_like(q)
        lse = torch.empty(R, Hq, device="cuda")
        pkt.check(pk.pk_attn_fwd(stream(), BF16, ptr(q), Hq * dk, ptr(k), Hkv * dk, ptr(v), Hkv * dk, ptr(out), Hq * dk,
                                 ptr(lse), B, S, Hq, Hkv, dk, scale, int(causal)))
        assert pk.pk_attn_last_path() == 1
        dq, dkk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        sc = scratch(pk.pk_attn_bwd_scratch_bytes(B, S, Hq))
        pkt.check(pk.pk_attn_bwd(stream(), BF16, ptr(q), Hq * dk, ptr(k), Hkv * dk, ptr(v), Hkv * dk, ptr(out), Hq * dk,
                                 ptr(lse), ptr(do), Hq * dk, ptr(dq), Hq * dk, ptr(dkk), Hkv * dk, ptr(dv), Hkv * dk, ptr(sc),
                                 B, S, Hq, Hkv, dk, scale, int(causal)))
        torch.cuda.synchronize()
        return [t[:(B - 1) * S].clone() for t in (out, lse, dq, dkk, dv)]

    clean, poisoned = run(False), run(True)
    for name, a, b in zip(("out", "lse", "dq", "dk", "dv"), clean, poisoned):
        assert bool(torch.isfinite(b.float()).all()), f"{name}: the neighbouring sequence leaked in"
        assert torch.equal(a, b), f"{name} of the untouched sequences changed"
    st = ctypes.c_int(0)
    pkt.check(pk.pk_attn_tc_status(ctypes.byref(st), 1))
    assert st.value == 0


@pytest.mark.parametrize("cfg", [(2, 200, 2, 2, 64, True), (1, 640, 4, 1, 64, True), (2, 333, 2, 2, 128, False),
                                 (1, 1100, 2, 2, 128, True)])
def test_attention_tensor_core_growing_maxima(pk, cfg):
    """The tcgen05 forward keeps the running output in tensor memory and rescales it only when a
    row maximum grows by more than 2^8; queries are scaled up and keys grow along the sequence so
    that row maxima keep growing and that rescale is exercised again and again. Forward and
    backward agree with the fp32 restatement of ops::fused_attention (src/ops.cpp:863-934), and
    the log-sum-exp agrees with the SIMT kernel's, which rescales on every tile."""
    B, S, Hq, Hkv, dk, causal = cfg
    R = B * S
    q = rnd(R, Hq * dk, seed=11, lo=-1, hi=1, dtype=torch.bfloat16) * 6
    k = rnd(R, Hkv * dk, seed=12, lo=-1, hi=1, dtype=torch.bfloat16)
    ramp = torch.linspace(0.2, 3.0, S, device="cuda").repeat(B).unsqueeze(1)
    k = (k.float() * ramp).to(torch.bfloat16)
    v = rnd(R, Hkv * dk, seed=13, lo=-1, hi=1, dtype=torch.bfloat16)
    do = rnd(R, Hq * dk, seed=14, lo=-1, hi=1, dtype=torch.bfloat16)
    scale = 1.0 / math.sqrt(dk)
    qf, kf, vf = (t.float().requires_grad_(True) for t in (q, k, v))
    ref = attn_ref(qf, kf, vf, B, S, Hq, Hkv, dk, scale, causal)
    ref.backward(do.float())
    lses = {}
    try:
        for simt in (0, 1):
            pkt.check(pk.pk_attn_force_simt(simt))
            out = torch.empty_like(q)
            lse = torch.empty(R, Hq, device="cuda")
            pkt.check(pk.pk_attn_fwd(stream(), dt(q), ptr(q), Hq * dk, ptr(k), Hkv * dk, ptr(v), Hkv * dk, ptr(out),
                                     Hq * dk, ptr(lse), B, S, Hq, Hkv, dk, scale, int(causal)))
            assert pk.pk_attn_last_path() == 1 - simt
            lses[simt] = lse
            if simt:
                continue
            dq, dkk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
            sc = scratch(pk.pk_attn_bwd_scratch_bytes(B, S, Hq))
            pkt.check(pk.pk_attn_bwd(stream(), dt(q), ptr(q), Hq * dk, ptr(k), Hkv * dk, ptr(v), Hkv * dk, ptr(out),
                                     Hq * dk, ptr(lse), ptr(do), Hq * dk, ptr(dq), Hq * dk, ptr(dkk), Hkv * dk,
                                     ptr(dv), Hkv * dk, ptr(sc), B, S, Hq, Hkv, dk, scale, int(causal)))
            st = ctypes.c_int(0)
            pkt.check(pk.pk_attn_tc_status(ctypes.byref(st), 1))
            assert st.value == 0, "a bounded wait gave up"
            close(out, ref, 2e-2, 2 ** -6)
            close(dq, qf.grad, 6e-2, 2 ** -5)
            close(dkk, kf.grad, 6e-2, 2 ** -5)
            close(dv, vf.grad, 6e-2, 2 ** -5)
    finally:
        pkt.check(pk.pk_attn_force_simt(0))
    close(lses[0], lses[1], 1e-3)


def test_attention_batch_isolation(pk):
    """Perturbing sequence 2 leaves sequence 1's output bitwise unchanged
    (tests/test_batching.cpp:108-120 of the reference asserts exactly 0.0)."""
    B, S, H, dk = 2, 48, 2, 32
    R = B * S
    q, k, v = (rnd(R, H * dk, seed=s, lo=-1, hi=1) for s in (1, 2, 3))

    def run(q, k, v):
        out = torch.empty_like(q)
        lse = torch.empty(R, H, device="cuda")
        pkt.check(pk.pk_attn_fwd(stream(), F32, ptr(q), H * dk, ptr(k), H * dk, ptr(v), H * dk, ptr(out), H * dk,
                                 ptr(lse), B, S, H, H, dk, 0.17, 1))
        return out

    a = run(q, k, v)
    k2, v2 = k.clone(), v.clone()
    k2[S:] += 1.0
    v2[S:] -= 2.0
    b = run(q, k2, v2)
    assert torch.equal(a[:S], b[:S])
    assert not torch.equal(a[S:], b[S:])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding_and_cross_entropy(pk, dtype):
    V, d, R = 50, 24, 40
    table = rnd(V, d, seed=1, dtype=dtype)
    g = torch.Generator().manual_seed(7)
    ids = torch.randint(0, V, (R,), generator=g, dtype=torch.int32).cuda()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = torch.empty(R, d, dtype=dtype, device="cuda")
    pkt.check(pk.pk_embedding_fwd(stream(), dt(table), ptr(table), ptr(ids), ptr(out), R, d, V, ptr(status)))
    assert torch.equal(out, table[ids.long()])  # pure copy: bit exact
    assert status.item() == 0
    bad = ids.clone()
    bad[3] = V + 4
    pkt.check(pk.pk_embedding_fwd(stream(), dt(table), ptr(table), ptr(bad), ptr(out), R, d, V, ptr(status)))
    assert status.item() == 5 and bool((out[3] == 0).all())
    # scatter-add in ascending position order == the reference's loop order
    dy = rnd(R, d, seed=2, dtype=dtype)
    ids_h = ids.cpu().numpy()
    order = np.argsort(ids_h, kind="stable").astype(np.int32)
    uniq, counts = np.unique(ids_h, return_counts=True)
    seg = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
    dtab = torch.zeros(V, d, device="cuda")
    # keep the index tensors referenced until the kernel has run
    order_d, seg_d = torch.from_numpy(order).cuda(), torch.from_numpy(seg).cuda()
    uniq_d = torch.from_numpy(uniq.astype(np.int32)).cuda()
    pkt.check(pk.pk_embedding_bwd(stream(), dt(dy), ptr(dy), ptr(order_d), ptr(seg_d), ptr(uniq_d),
                                  len(uniq), ptr(dtab), d))
    ref = np.zeros((V, d), dtype=np.float32)
    dyh = dy.float().cpu().numpy()
    for i in range(R):
        ref[ids_h[i]] += dyh[i]
    assert np.array_equal(dtab.cpu().numpy(), ref)  # same order, same bits
    # cross entropy
    for (Rr, Vv) in ((40, 24), (9, 4096), (5, 1000 + 3)):
        logits = rnd(Rr, Vv, seed=3, lo=-4, hi=4, dtype=dtype)
        tg = torch.randint(0, Vv, (Rr,), generator=g, dtype=torch.int32).cuda()
        lf = logits.float()
        P = torch.softmax(lf, dim=1)
        ar = torch.arange(Rr, device="cuda")
        ref_rows = -torch.log(torch.clamp(P[ar, tg.long()], min=1e-12))
        work = logits.clone()
        rows = torch.empty(Rr, device="cuda")
        status.zero_()
        pkt.check(pk.pk_cross_entropy(stream(), dt(work), ptr(work), Vv, ptr(tg), ptr(rows), Rr, Vv, 1.0 / Rr, 1,
                                      ptr(status)))
        close(rows, ref_rows, 2e-5, 1e-5)
        dref = P.clone()
        dref[ar, tg.long()] -= 1.0
        tol = 1e-6 if dtype == torch.float32 else 1e-3
        close(work, dref / Rr, tol, 0 if dtype == torch.float32 else 2 ** -7)
        total = torch.zeros(1, dtype=torch.float64, device="cuda")
        pkt.check(pk.pk_reduce_sum_f64(stream(), ptr(rows), Rr, 0, 0, ptr(total), ptr(scratch(pk.pk_reduce_scratch_bytes()))))
        assert abs(total.item() - rows.double().sum().item()) < 1e-9


def test_reduce_and_adamw(pk):
    n = 100003
    x = rnd(n, seed=1)
    out = torch.zeros(1, dtype=torch.float64, device="cuda")
    sc = scratch(pk.pk_reduce_scratch_bytes())
    pkt.check(pk.pk_reduce_sum_f64(stream(), ptr(x), n, 1, 0, ptr(out), ptr(sc)))
    assert abs(out.item() - (x.double() ** 2).sum().item()) < 1e-6
    pkt.check(pk.pk_reduce_sum_f64(stream(), ptr(x), n, 1, 1, ptr(out), ptr(sc)))
    assert abs(out.item() - 2 * (x.double() ** 2).sum().item()) < 1e-6
    # AdamW: three steps, fp32 formula of AdamW::step (src/nn.cpp:301-321)
    p = rnd(1001, seed=2)
    m = torch.zeros_like(p)
    v = torch.zeros_like(p)
    shadow = torch.empty(1001, dtype=torch.bfloat16, device="cuda")
    pr, mr, vr = p.clone(), m.clone(), v.clone()
    lr, b1, b2, eps, wd = 1e-3, 0.9, 0.999, 1e-8, 0.01
    for t in range(1, 4):
        g = rnd(1001, seed=10 + t)
        c1 = float(np.float32(1) - np.float32(np.power(np.float32(b1), np.float32(t))))
        c2 = float(np.float32(1) - np.float32(np.power(np.float32(b2), np.float32(t))))
        pkt.check(pk.pk_adamw(stream(), ptr(p), ptr(g), ptr(m), ptr(v), 1001, lr, b1, b2, eps, wd, c1, c2, ptr(shadow)))
        mr = b1 * mr + (1 - b1) * g
        vr = b2 * vr + (1 - b2) * g * g
        pr = pr - lr * ((mr / c1) / (torch.sqrt(vr / c2) + eps) + wd * pr)
        close(p, pr, 1e-6)
        assert torch.equal(shadow, p.to(torch.bfloat16))


def test_q8_roundtrip(pk):
    rows, cols = 24, 96
    W = rnd(rows, cols, seed=1, lo=-1, hi=1)
    W[3, :32] = 0.0
    q = torch.empty(rows, cols, dtype=torch.int8, device="cuda")
    sc = torch.empty(rows, cols // 32, dtype=torch.float16, device="cuda")
    pkt.check(pk.pk_q8_quantize(stream(), ptr(W), ptr(q), ptr(sc), rows, cols))
    Wb = W.view(rows, cols // 32, 32)
    amax = Wb.abs().amax(dim=2)
    s = torch.where(amax > 0, amax / 127.0, torch.ones_like(amax)).to(torch.float16)
    assert torch.equal(sc, s)
    qr = torch.clamp(Wb / s.float()[:, :, None], -127, 127)
    qr = torch.where(qr >= 0, torch.floor(qr + 0.5), torch.ceil(qr - 0.5)).to(torch.int8).view(rows, cols)
    assert torch.equal(q, qr)
    deq = torch.empty(rows, cols, device="cuda")
    pkt.check(pk.pk_q8_dequantize(stream(), ptr(q), ptr(sc), F32, ptr(deq), rows, cols))
    assert torch.equal(deq, (q.float().view(rows, cols // 32, 32) * s.float()[:, :, None]).view(rows, cols))
    # half-step error bound of the reference's test (tests/test_lora_quant.cpp:37-54)
    err = (deq - W).abs().view(rows, cols // 32, 32)
    assert bool((err <= 0.5 * s.float()[:, :, None] + 1e-7).all())
    deqb = torch.empty(rows, cols, dtype=torch.bfloat16, device="cuda")
    pkt.check(pk.pk_q8_dequantize(stream(), ptr(q), ptr(sc), BF16, ptr(deqb), rows, cols))
    assert torch.equal(deqb, deq.to(torch.bfloat16))


def test_q8_block_quantisation_any_block(pk):
    """The reference's quantize_int8 / dequantize (src/quant.cpp:11-48) at its default block of 64
    and at a block length that leaves a short last block: fp32 scales, bit-exact."""
    rows, cols = 24, 100
    W = rnd(rows, cols, seed=2, lo=-1, hi=1)
    W[5, :64] = 0.0
    for block in (64, 48, 7):
        bpr = (cols + block - 1) // block
        q = torch.empty(rows, cols, dtype=torch.int8, device="cuda")
        sc = torch.empty(rows, bpr, device="cuda")
        pkt.check(pk.pk_q8_quantize_block(stream(), ptr(W), ptr(q), ptr(sc), rows, cols, block))
        pad = bpr * block - cols
        Wp = torch.nn.functional.pad(W, (0, pad)).view(rows, bpr, block)
        amax = Wp.abs().amax(dim=2)
        # IEEE division on the host: torch's division by a Python scalar multiplies by 1/127 on the GPU
        s_np = amax.cpu().numpy() / np.float32(127.0)
        s = torch.where(amax > 0, torch.from_numpy(s_np).cuda(), torch.ones_like(amax))
        assert torch.equal(sc, s)
        qr = torch.clamp(Wp / s[:, :, None], -127, 127)
        qr = torch.where(qr >= 0, torch.floor(qr + 0.5), torch.ceil(qr - 0.5)).to(torch.int8).view(rows, bpr * block)
        assert torch.equal(q, qr[:, :cols].contiguous())
        ref = (qr.float().view(rows, bpr, block) * s[:, :, None]).view(rows, bpr * block)[:, :cols].contiguous()
        for odt, tdt in ((F32, torch.float32), (BF16, torch.bfloat16)):
            deq = torch.empty(rows, cols, dtype=tdt, device="cuda")
            pkt.check(pk.pk_q8_dequantize_block(stream(), ptr(q), ptr(sc), block, odt, ptr(deq), rows, cols))
            assert torch.equal(deq, ref.to(tdt))
        err = (ref - W).abs().view(rows, cols)
        lim = torch.repeat_interleave(0.5 * s, block, dim=1)[:, :cols]
        assert bool((err <= lim + 1e-7).all())


def q8_weight(pk, rows, cols, seed):
    W = rnd(rows, cols, seed=seed, lo=-0.06, hi=0.06)
    q = torch.empty(rows, cols, dtype=torch.int8, device="cuda")
    sc = torch.empty(rows, cols // 32, dtype=torch.float16, device="cuda")
    pkt.check(pk.pk_q8_quantize(stream(), ptr(W), ptr(q), ptr(sc), rows, cols))
    deq = torch.empty(rows, cols, dtype=torch.bfloat16, device="cuda")
    pkt.check(pk.pk_q8_dequantize(stream(), ptr(q), ptr(sc), BF16, ptr(deq), rows, cols))
    return q, sc, deq


def q8_call(pk, trans_w, A, q, sc, M, N, K, XA=None, L=None, C=None, out_dtype=torch.bfloat16, accumulate=False,
            bias=None, residual=None):
    if C is None:
        C = torch.empty(M, N, dtype=out_dtype, device="cuda")
    r = 0 if XA is None else XA.shape[1]
    pkt.check(pk.pk_gemm_q8_lora(stream(), dt(C), int(trans_w), M, N, K, ptr(A), A.stride(0), ptr(q), ptr(sc),
                                 ptr(XA), XA.stride(0) if XA is not None else 0, ptr(L),
                                 L.stride(0) if L is not None else 0, r, ptr(C), C.stride(0), int(accumulate),
                                 ptr(bias), ptr(residual), residual.stride(0) if residual is not None else 0),
              "pk_gemm_q8_lora")
    assert pk.pk_gemm_last_path() == 4
    return C


# (M, N, K); sized so that the dense comparison GEMM never takes split-K, whose summation order differs
@pytest.mark.parametrize("shape", [(300, 896, 896), (1024, 128, 896), (1500, 4864, 896), (1501, 896, 4864), (64, 128, 40),
                                   (4096, 896, 896)])
@pytest.mark.parametrize("rank", [0, 16, 8, 64])
def test_gemm_q8_lora_equals_dequantise_then_gemm(pk, shape, rank):
    """The fused kernel forms the products of a bf16 GEMM over the expanded weight in the same k
    order: y = x deq(W) + XA B equals pk_gemm([x | XA], [deq(W); B]) BIT FOR BIT, and so does the
    input-gradient form dx = dy deq(W)^T + DXA A^T. (src/quant.cpp:91-119 is the layer this
    replaces; the reference multiplies by a dequantised copy.) Also against fp32 torch."""
    M, N, K = shape
    # forward: W is [K, N]
    q, sc, deq = q8_weight(pk, K, N, seed=3)
    x = rnd(M, K, seed=4, dtype=torch.bfloat16)
    xa = rnd(M, rank, seed=5, lo=-0.5, hi=0.5, dtype=torch.bfloat16) if rank else None
    Bl = rnd(rank, N, seed=6, lo=-0.05, hi=0.05, dtype=torch.bfloat16) if rank else None
    res = rnd(M, N, seed=7, dtype=torch.bfloat16)
    y = q8_call(pk, 0, x, q, sc, M, N, K, xa, Bl, residual=res)
    if rank:
        unfused = pkt.gemm(torch.cat([x, xa], dim=1).contiguous(), torch.cat([deq, Bl], dim=0).contiguous(), residual=res)
    else:
        unfused = pkt.gemm(x, deq, residual=res)
    assert pk.pk_gemm_last_path() in (2, 3)
    # (with a k extent that is not a multiple of 16 the concatenated operands group the products of
    # the last steps differently; the bitwise claim is for whole 16-deep steps)
    if rank == 0 or K % 16 == 0:
        assert torch.equal(y, unfused), f"forward differs: max {(y.float() - unfused.float()).abs().max().item():.3e}"
    ref = x.float() @ deq.float() + res.float()
    if rank:
        ref = ref + xa.float() @ Bl.float()
    close(y, ref, 2e-2, 2 ** -6)
    # input gradient: dy [M, N] . deq(W)^T -> [M, K]; the LoRA operand is A [K, r]
    dy = rnd(M, N, seed=8, dtype=torch.bfloat16)
    dxa = rnd(M, rank, seed=9, lo=-0.5, hi=0.5, dtype=torch.bfloat16) if rank else None
    Al = rnd(K, rank, seed=10, lo=-0.05, hi=0.05, dtype=torch.bfloat16) if rank else None
    dx = q8_call(pk, 1, dy, q, sc, M, K, N, dxa, Al)
    if rank:
        unfused = pkt.gemm(torch.cat([dy, dxa], dim=1).contiguous(), torch.cat([deq, Al], dim=1).contiguous(), tb=True)
    else:
        unfused = pkt.gemm(dy, deq, tb=True)
    assert torch.equal(dx, unfused), f"input gradient differs: max {(dx.float() - unfused.float()).abs().max().item():.3e}"
    # accumulate into an existing gradient, fp32 output, and a bias
    bias = rnd(K, seed=11)
    acc0 = rnd(M, K, seed=12)
    acc = acc0.clone()
    q8_call(pk, 1, dy, q, sc, M, K, N, dxa, Al, C=acc, accumulate=True, bias=bias)
    ref = acc0 + dy.float() @ deq.float().T + bias[None, :]
    if rank:
        ref = ref + dxa.float() @ Al.float().T
    close(acc, ref, 2e-2, 1e-3)
    st = ctypes.c_int(0)
    pkt.check(pk.pk_gemm_tc_status(ctypes.byref(st), 1))
    assert st.value == 0, "a bounded wait gave up"
    # repeatable bit for bit
    assert torch.equal(y, q8_call(pk, 0, x, q, sc, M, N, K, xa, Bl, residual=res))


def test_gemm_q8_rejects_what_it_does_not_take(pk):
    q, sc, _ = q8_weight(pk, 64, 64, seed=1)
    x = rnd(16, 64, seed=2, dtype=torch.bfloat16)
    y = torch.empty(16, 64, dtype=torch.bfloat16, device="cuda")
    xa = rnd(16, 12, seed=3, dtype=torch.bfloat16)   # rank not a multiple of 8
    L = rnd(12, 64, seed=4, dtype=torch.bfloat16)
    rc = pk.pk_gemm_q8_lora(stream(), BF16, 0, 16, 64, 64, ptr(x), 64, ptr(q), ptr(sc), ptr(xa), 12, ptr(L), 64, 12,
                            ptr(y), 64, 0, None, None, 0)
    assert rc == 3  # PK_ERR_UNSUPPORTED
    rc = pk.pk_gemm_q8_lora(stream(), BF16, 0, 16, 64, 64, ptr(x), 32, ptr(q), ptr(sc), None, 0, None, 0, 0, ptr(y), 64,
                            0, None, None, 0)
    assert rc == 1  # PK_ERR_INVALID: lda < K
    rc = pk.pk_gemm_q8_lora(stream(), BF16, 0, 16, 64, 64, ptr(x), 64, ptr(q), ptr(sc), None, 0, None, 0, 0, ptr(y), 64,
                            0, None, None, 0)
    assert rc == 3  # PK_ERR_UNSUPPORTED: 64 columns of W, the kernel wants a multiple of 128


def test_bounded_wait_runs_out_and_the_library_carries_on(pk):
    """A wait on an mbarrier nobody arrives at gives up at the limit, records PK_ERR_TIMEOUT and
    the kernel returns; nothing traps, the context stays usable and the kernels' own status words
    stay clean. The limit is settable (default 2 s)."""
    import time
    try:
        pkt.check(pk.pk_set_wait_limit_us(2000.0))
        st = ctypes.c_int(0)
        waited = ctypes.c_double(0.0)
        t0 = time.perf_counter()
        pkt.check(pk.pk_wait_selftest(stream(), ctypes.byref(st), ctypes.byref(waited)))
        wall = time.perf_counter() - t0
        assert st.value == 4, f"status {st.value}, expected PK_ERR_TIMEOUT"
        assert 2000.0 <= waited.value < 200000.0, waited.value
        assert wall < 1.0
        # the word was cleared by the read
        pkt.check(pk.pk_set_wait_limit_us(500.0))
        pkt.check(pk.pk_wait_selftest(stream(), ctypes.byref(st), ctypes.byref(waited)))
        assert st.value == 4 and 500.0 <= waited.value < 100000.0
    finally:
        pkt.check(pk.pk_set_wait_limit_us(2e6))
    # normal work afterwards: tensor-core GEMM and attention, correct and with clean status
    a = rnd(512, 256, seed=1, dtype=torch.bfloat16)
    b = rnd(256, 512, seed=2, dtype=torch.bfloat16)
    c = pkt.gemm(a, b)
    assert pk.pk_gemm_last_path() in (2, 3)
    close(c, a.float() @ b.float(), 0.5, 2 ** -6)
    B, S, H, dk = 1, 256, 2, 64
    qq = rnd(S, H * dk, seed=3, lo=-1, hi=1, dtype=torch.bfloat16)
    out = torch.empty_like(qq)
    lse = torch.empty(S, H, device="cuda")
    pkt.check(pk.pk_attn_fwd(stream(), BF16, ptr(qq), H * dk, ptr(qq), H * dk, ptr(qq), H * dk, ptr(out), H * dk, ptr(lse),
                             B, S, H, H, dk, 0.125, 1))
    assert pk.pk_attn_last_path() == 1
    ref = attn_ref(qq.float(), qq.float(), qq.float(), B, S, H, H, dk, 0.125, True)
    close(out, ref, 2e-2, 2 ** -6)
    all_st = ctypes.c_int(-1)
    pkt.check(pk.pk_device_sync())
    pkt.check(pk.pk_kernel_status(ctypes.byref(all_st), 1))
    assert all_st.value == 0


@pytest.mark.parametrize("shape", [(300, 128, 64), (1024, 4864, 896), (2048, 8192, 2048), (515, 136, 72)])
def test_gemm_swiglu_equals_the_three_separate_calls(pk, shape):
    """y = silu(x Wg) .* (x Wu) from the one-pass kernel has the bits of pk_gemm + pk_gemm +
    pk_swiglu_fwd, with or without G and U being stored (src/llama.cpp:55-58 of the reference is the
    composition it replaces)."""
    M, N, K = shape
    x = rnd(M, K, seed=1, dtype=torch.bfloat16)
    Wg = rnd(K, N, seed=2, lo=-0.1, hi=0.1, dtype=torch.bfloat16)
    Wu = rnd(K, N, seed=3, lo=-0.1, hi=0.1, dtype=torch.bfloat16)
    G_ref, U_ref = pkt.gemm(x, Wg), pkt.gemm(x, Wu)
    y_ref = torch.empty_like(G_ref)
    pkt.check(pk.pk_swiglu_fwd(stream(), BF16, ptr(G_ref), ptr(U_ref), ptr(y_ref), M * N))
    for keep in (True, False):
        G = torch.full((M, N), 7.0, dtype=torch.bfloat16, device="cuda") if keep else None
        U = torch.full((M, N), 7.0, dtype=torch.bfloat16, device="cuda") if keep else None
        y = torch.full((M, N), 7.0, dtype=torch.bfloat16, device="cuda")
        pkt.check(pk.pk_gemm_swiglu(stream(), M, N, K, ptr(x), K, ptr(Wg), N, ptr(Wu), N, ptr(G), ptr(U), N, ptr(y), N),
                  "pk_gemm_swiglu")
        assert pk.pk_gemm_last_path() == 3
        assert torch.equal(y, y_ref), f"y differs (keep={keep}): max {(y.float() - y_ref.float()).abs().max().item():.3e}"
        if keep:
            assert torch.equal(G, G_ref) and torch.equal(U, U_ref)
    gf, uf = G_ref.float(), U_ref.float()
    close(y_ref, gf / (1 + torch.exp(-gf)) * uf, 1e-2, 2 ** -7)
    st = ctypes.c_int(0)
    pkt.check(pk.pk_gemm_tc_status(ctypes.byref(st), 1))
    assert st.value == 0
    # shapes the kernel does not take are reported, not mangled
    assert pk.pk_gemm_swiglu(stream(), 64, N, K, ptr(x), K, ptr(Wg), N, ptr(Wu), N, None, None, N, ptr(y), N) == 3


@pytest.mark.parametrize("shape", [(4096, 2048, 512, 64, 32, False, False), (16384, 512, 264, 64, 1, True, False),
                                   (2048, 4096, 384, 128, 16, False, True), (4099, 2048, 512, 64, 12, False, True)])
def test_gemm_rope_equals_gemm_then_rope(pk, shape):
    """pk_gemm_rope (the q / k projection with the rotary embedding applied in the GEMM's epilogue)
    gives pk_gemm followed by pk_rope bit for bit: all heads or only the first, both layouts of
    the weight, with a bias, ragged rows, forward and inverse rotation. Shapes the kernel does not
    take are refused with PK_ERR_UNSUPPORTED."""
    M, N, K, hd, nh, tb, with_bias = shape
    A = rnd(M, K, seed=1, lo=-1, hi=1, dtype=torch.bfloat16)
    B = rnd(N, K, seed=2, lo=-1, hi=1, dtype=torch.bfloat16) if tb else rnd(K, N, seed=2, lo=-1, hi=1, dtype=torch.bfloat16)
    bias = rnd(1, N, seed=3).reshape(N) if with_bias else None
    n_pos = 777
    pos = torch.tensor([(7 * i) % n_pos for i in range(M)], dtype=torch.int32, device="cuda")
    j = np.arange(hd // 2, dtype=np.float32)
    inv = (np.float32(1.0) / np.power(np.float32(10000.0), (2 * j) / np.float32(hd))).astype(np.float32)
    th = np.arange(n_pos, dtype=np.float32)[:, None] * inv[None, :]
    tab = torch.from_numpy(np.stack([np.cos(th), np.sin(th)], axis=-1).astype(np.float32)).cuda().contiguous()
    for inverse in (0, 1):
        two = pkt.gemm(A, B, tb=tb, bias=bias)
        pkt.check(pk.pk_rope(stream(), dt(two), ptr(two), N, 0, nh, hd, ptr(pos), ptr(tab), n_pos, M, inverse))
        one = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
        pkt.check(pk.pk_gemm_rope(stream(), int(tb), M, N, K, ptr(A), K, ptr(B), B.stride(0), ptr(one), N, ptr(bias),
                                  ptr(pos), ptr(tab), n_pos, nh, hd, inverse))
        assert pk.pk_gemm_last_path() == 3
        assert torch.equal(one, two), (one.float() - two.float()).abs().max()
    st = ctypes.c_int(0)
    pkt.check(pk.pk_gemm_tc_status(ctypes.byref(st), 1))
    assert st.value == 0
    # head_dim 32: a 32-column unit would span two heads
    rc = pk.pk_gemm_rope(stream(), int(tb), M, N, K, ptr(A), K, ptr(B), B.stride(0), ptr(one), N, None, ptr(pos), ptr(tab),
                         n_pos, 1, 32, 0)
    assert rc == 3  # PK_ERR_UNSUPPORTED
    # too few rows for the pair kernel
    rc = pk.pk_gemm_rope(stream(), int(tb), 64, N, K, ptr(A), K, ptr(B), B.stride(0), ptr(one), N, None, ptr(pos), ptr(tab),
                         n_pos, nh, hd, 0)
    assert rc == 3

