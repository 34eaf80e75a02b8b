"""Helpers for the kernel-level GPU tests: call libpk entry points on torch tensors."""
import ctypes

import torch

from paperkiln_b200._capi import check, libpk

F32, BF16 = 0, 1


def dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise TypeError(t.dtype)


def ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


_live = []


def scratch(nbytes: int) -> torch.Tensor:
    # filled with garbage on purpose: results must not depend on scratch contents.
    # The tensor stays referenced (until release()) so that its memory cannot be handed
    # to another allocation while a kernel still uses it.
    t = torch.full((max(int(nbytes), 16),), 0x5A, dtype=torch.uint8, device="cuda")
    _live.append(t)
    return t


def release():
    torch.cuda.synchronize()
    _live.clear()


def gemm(A, B, *, ta=False, tb=False, out_dtype=None, C=None, accumulate=False, bias=None,
         residual=None):
    pk = libpk()
    M = A.shape[1] if ta else A.shape[0]
    K = A.shape[0] if ta else A.shape[1]
    N = B.shape[0] if tb else B.shape[1]
    out_dtype = out_dtype or A.dtype
    if C is None:
        C = torch.empty(M, N, dtype=out_dtype, device="cuda")
    check(pk.pk_gemm(stream(), dt(A), dt(C), int(ta), int(tb), M, N, K, ptr(A), A.stride(0),
                     ptr(B), B.stride(0), ptr(C), C.stride(0), int(accumulate), ptr(bias),
                     ptr(residual), residual.stride(0) if residual is not None else 0), "pk_gemm")
    return C
