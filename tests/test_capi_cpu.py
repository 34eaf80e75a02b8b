"""The shared libraries load on a machine without a GPU and export every symbol the headers
under include/ declare; GPU-free host logic (spec parsing, error reporting, sharding)."""
import ctypes
from pathlib import Path

import numpy as np
import pytest

from paperkiln_b200 import _capi, dp

ROOT = Path(__file__).resolve().parent.parent


def test_headers_parse_and_symbols_exported():
    pk = _capi.libpk()
    mt = _capi.libmt()
    assert len(pk.protos) >= 60 and len(mt.protos) >= 24
    for lib, header in ((pk, ROOT / "include" / "pk.h"), (mt, ROOT / "include" / "mt_capi.h")):
        declared = _capi.parse_header(header)
        for name in declared:
            assert hasattr(lib.dll, name), f"{lib.path.name} does not export {name}"
    assert pk.pk_abi_version() == 1


def test_no_silent_cpu_fallback():
    """Without a GPU every entry that needs one fails with an error code and a message."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    mt = _capi.libmt()
    assert mt.mt_init(0, 0) != 0
    assert b"pk_device_count" in mt.mt_last_error() or b"CUDA" in mt.mt_last_error()
    h = ctypes.c_void_p()
    assert mt.mt_model_create(b"family=llama;vocab=16;d=8;layers=1;heads=2;dff=16", ctypes.byref(h)) != 0
    assert b"no CPU fallback" in mt.mt_last_error() or b"CUDA" in mt.mt_last_error()


def test_argument_validation_needs_no_gpu():
    pk = _capi.libpk()
    # bad dtype / negative sizes are rejected before any CUDA call
    assert pk.pk_gelu_fwd(None, 7, None, None, 4) == 1
    assert b"dtype" in pk.pk_last_error()
    assert pk.pk_gemm(None, 0, 0, 0, 0, -1, 2, 2, None, 2, None, 2, None, 2, 0, None, None, 0) == 1
    assert pk.pk_q8_quantize(None, None, None, None, 4, 33) == 1
    assert pk.pk_rope(None, 0, None, 8, 0, 1, 3, None, None, 1, 4, 0) == 1  # odd head_dim
    # empty work is accepted
    assert pk.pk_gelu_fwd(None, 0, None, None, 0) == 0
    assert pk.pk_attn_fwd(None, 0, None, 8, None, 8, None, 8, None, 8, None, 0, 0, 1, 1, 8, 1.0, 1) == 0


def test_model_spec_errors():
    mt = _capi.libmt()
    h = ctypes.c_void_p()
    assert mt.mt_model_create(b"family=llama;bogus=1", ctypes.byref(h)) != 0
    assert b"unknown key" in mt.mt_last_error() or b"CUDA" in mt.mt_last_error() or b"fallback" in mt.mt_last_error()
    assert mt.mt_model_create(b"family=transformerxl", ctypes.byref(h)) != 0


def test_sharding():
    stream = np.arange(4 * 6 + 1, dtype=np.int32)
    parts = [dp.shard_tokens(stream, 4, 6, r, 2) for r in range(2)]
    assert np.array_equal(np.concatenate([p[0] for p in parts]), stream[:-1])
    assert np.array_equal(np.concatenate([p[1] for p in parts]), stream[1:])
    assert dp.shard_range(8, 3, 4) == (6, 8)
    with pytest.raises(ValueError):
        dp.shard_range(6, 0, 4)
    with pytest.raises(ValueError):
        dp.shard_tokens(stream[:-1], 4, 6, 0, 2)
