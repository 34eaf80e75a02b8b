"""pk_rmsnorm_bwd_noalloc: the RMSNorm backward for hosts that cannot allocate device memory
(a runtime that already owns the whole GPU, or a loop that must not hit cudaMalloc's device
synchronisation). It keeps its partial sums in a buffer built into the library instead of
caller-provided scratch. Checked here against pk_rmsnorm_bwd on the same inputs: the results
must be the same bits, on two calls in a row (the second with another shape, so that whatever
the first call left in the shared buffer is shown not to matter), and sizes beyond the
built-in buffer must be refused with a message. Collected last on purpose (file name)."""
import ctypes

import pytest
import torch

from tests import pkt
from tests.pkt import dt, ptr, scratch, stream

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def pk():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from paperkiln_b200._capi import libpk
    return libpk()


def _inputs(R, C, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    x = (torch.rand(R, C, generator=g) * 3 - 1.5).to(dtype).cuda()
    dy = (torch.rand(R, C, generator=g) * 2 - 1).to(dtype).cuda()
    w = (torch.rand(C, generator=g) + 0.5).cuda()
    y = torch.empty_like(x)
    rinv = torch.empty(R, device="cuda")
    pkt.check(libpk_().pk_rmsnorm_fwd(stream(), dt(x), ptr(x), ptr(w), ptr(y), ptr(rinv), R, C, 1e-5))
    return x, dy, w, rinv


def libpk_():
    from paperkiln_b200._capi import libpk
    return libpk()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_noalloc_matches_scratch_version_twice(pk, dtype):
    for call, (R, C) in enumerate([(300, 768), (67, 133), (1000, 2048)]):
        x, dy, w, rinv = _inputs(R, C, dtype, seed=10 + call)
        dx_ref = torch.empty_like(x)
        dw_ref = torch.full((C,), 0.5, device="cuda")
        sc = scratch(pk.pk_rmsnorm_bwd_scratch_bytes(R, C))
        pkt.check(pk.pk_rmsnorm_bwd(stream(), dt(x), ptr(dy), ptr(x), ptr(w), ptr(rinv), ptr(dx_ref), ptr(dw_ref),
                                    ptr(sc), R, C))
        dx = torch.empty_like(x)
        dw = torch.full((C,), 0.5, device="cuda")
        pkt.check(pk.pk_rmsnorm_bwd_noalloc(stream(), dt(x), ptr(dy), ptr(x), ptr(w), ptr(rinv), ptr(dx), ptr(dw), R, C))
        assert torch.equal(dx, dx_ref), f"call {call}: dx differs"
        assert torch.equal(dw, dw_ref), f"call {call}: dw differs"


def test_noalloc_rejects_oversize(pk):
    R, C = 4, 8192  # beyond the built-in buffer on a 148-SM GPU
    if pk.pk_rmsnorm_bwd_scratch_bytes(R, C) <= 592 * 4096 * 4:
        pytest.skip("this GPU has few enough SMs for C = 8192 to fit")
    x = torch.zeros(R, C, device="cuda")
    w = torch.ones(C, device="cuda")
    rinv = torch.ones(R, device="cuda")
    dw = torch.zeros(C, device="cuda")
    rc = pk.pk_rmsnorm_bwd_noalloc(stream(), 0, ptr(x), ptr(x), ptr(w), ptr(rinv), ptr(x), ptr(dw), R, C)
    assert rc == 3
    assert b"built-in buffer" in pk.pk_last_error()
