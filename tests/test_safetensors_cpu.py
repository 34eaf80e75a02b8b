"""Checkpoint file format on CPU: the host library's safetensors reader / writer against the
layout and the loader rules of the reference (src/safetensors.cpp:12-94): 8-byte little-endian
header length, JSON header, fp32 tensors in sorted name order, header padded to 8 bytes; tensors
of rank > 2 skipped, a leading "transformer." stripped, "__metadata__" ignored, [n] -> [1, n].
The files are written and read back here with numpy and the json module; no GPU is involved."""
import ctypes
import json
import struct

import numpy as np
import pytest

from paperkiln_b200._capi import libmt


def write_file(path, tensors, metadata=None):
    """tensors: list of (name, dtype string, array). Keys in the given order (not sorted)."""
    header, blobs, off = {}, [], 0
    if metadata is not None:
        header["__metadata__"] = metadata
    for name, dtype, arr in tensors:
        raw = arr.tobytes()
        header[name] = {"dtype": dtype, "shape": list(arr.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    text = json.dumps(header).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(text)))
        f.write(text)
        for b in blobs:
            f.write(b)


def read_file(path):
    raw = open(path, "rb").read()
    (hlen,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + hlen].decode())
    out = {}
    for name, meta in header.items():
        lo, hi = meta["data_offsets"]
        assert meta["dtype"] == "F32"
        out[name] = np.frombuffer(raw[8 + hlen + lo:8 + hlen + hi], dtype="<f4").reshape(meta["shape"])
    return hlen, list(header.keys()), out, raw


def to_bf16_bits(x):
    return (x.astype("<f4").view("<u4") >> 16).astype("<u2")


def copy(src, dst):
    n, k = ctypes.c_int64(-1), ctypes.c_int64(-1)
    rc = libmt().mt_safetensors_copy(str(src).encode(), str(dst).encode(), ctypes.byref(n), ctypes.byref(k))
    return rc, n.value, k.value


def test_loader_rules_and_writer_layout(tmp_path):
    rng = np.random.RandomState(5)
    w = rng.randn(7, 12).astype("<f4")
    b = rng.randn(12).astype("<f4")
    h = rng.randn(4, 6).astype("<f4")
    mask = np.ones((1, 1, 8, 8), dtype="<f4")
    scalar = np.array(3.5, dtype="<f4")
    src, dst = tmp_path / "in.safetensors", tmp_path / "out.safetensors"
    write_file(src, [("zeta.weight", "F32", w), ("transformer.h.0.bias", "F32", b),
                     ("half \\\"quoted\\\"", "BF16", to_bf16_bits(h)), ("h.0.attn.bias", "F32", mask),
                     ("alpha", "F32", scalar)], metadata={"format": "pt", "nested": {"k": [1, 2.5, None, True]}})
    rc, n, k = copy(src, dst)
    assert rc == 0, libmt().mt_last_error()
    assert (n, k) == (4, 1)
    hlen, names, out, raw = read_file(dst)
    assert hlen % 8 == 0 and raw[8:8 + hlen].rstrip(b" ")[-1:] == b"}"
    assert names == sorted(names) == ["alpha", "h.0.bias", "half \\\"quoted\\\"", "zeta.weight"]
    assert out["alpha"].shape == (1, 1) and out["alpha"][0, 0] == 3.5
    assert out["h.0.bias"].shape == (1, 12) and np.array_equal(out["h.0.bias"][0], b)
    assert np.array_equal(out["zeta.weight"], w)
    widened = (to_bf16_bits(h).astype("<u4") << 16).view("<f4").reshape(4, 6)
    assert np.array_equal(out["half \\\"quoted\\\""], widened)
    # data region: tensors back to back in the header's order
    total = sum(a.size for a in out.values()) * 4
    assert len(raw) == 8 + hlen + total
    # identical contents give identical bytes
    dst2 = tmp_path / "out2.safetensors"
    assert copy(dst, dst2)[0] == 0
    assert open(dst2, "rb").read() == raw


@pytest.mark.parametrize("case", ["dtype", "size", "truncated", "garbage", "missing", "huge_shape", "wrapping_shape"])
def test_loader_rejects_bad_files(tmp_path, case):
    src, dst = tmp_path / "bad.safetensors", tmp_path / "out.safetensors"
    x = np.arange(6, dtype="<f4").reshape(2, 3)
    if case == "dtype":
        write_file(src, [("x", "I64", x.astype("<i8"))])
    elif case == "size":
        write_file(src, [("x", "F32", x)])
        raw = bytearray(open(src, "rb").read())
        raw = raw.replace(b"[2, 3]", b"[2, 4]")
        open(src, "wb").write(raw)
    elif case == "truncated":
        write_file(src, [("x", "F32", x)])
        raw = open(src, "rb").read()
        open(src, "wb").write(raw[:-8])
    elif case in ("huge_shape", "wrapping_shape"):
        # a hostile header: the claimed shape would need an enormous allocation, or its byte count
        # wraps around 2^64 to the 24 bytes that are really there -- rejected before any allocation
        write_file(src, [("x", "F32", x)])
        raw = bytearray(open(src, "rb").read())
        claim = b"[4611686018427387904, 3]" if case == "huge_shape" else b"[4611686018427387905, 4]"
        hlen = struct.unpack("<Q", raw[:8])[0]
        head = bytes(raw[8:8 + hlen]).replace(b"[2, 3]", claim)
        head += b" " * ((-len(head)) % 8)
        open(src, "wb").write(struct.pack("<Q", len(head)) + head + bytes(raw[8 + hlen:]))
    elif case == "garbage":
        open(src, "wb").write(struct.pack("<Q", 16) + b"{\"x\": [1, 2, }  ")
    else:
        src = tmp_path / "does_not_exist.safetensors"
    rc, _, _ = copy(src, dst)
    assert rc != 0
    assert b"safetensors" in libmt().mt_last_error()


def test_writer_matches_reference_bytes(tmp_path):
    """tests/golden/ref_writer.safetensors was written by the unmodified reference
    (save_safetensors, src/safetensors.cpp:60-94; generator: tests/golden/safetensors_ref_writer.cpp).
    Loading it and writing it back here gives the same bytes, and the values are the seeded ones."""
    from pathlib import Path
    gold = Path(__file__).resolve().parent / "golden" / "ref_writer.safetensors"
    dst = tmp_path / "copy.safetensors"
    rc, n, k = copy(gold, dst)
    assert rc == 0 and (n, k) == (2, 0)
    assert open(dst, "rb").read() == open(gold, "rb").read()
    rng = np.random.RandomState(1)
    w = rng.randn(5, 9).astype("<f4")
    b = rng.randn(9).astype("<f4")
    _, names, out, _ = read_file(dst)
    assert names == ["final_norm.weight", "layers.0.wq"]
    assert np.array_equal(out["layers.0.wq"], w) and np.array_equal(out["final_norm.weight"][0], b)
