"""ctypes bindings generated from the C headers under ``include/``.

The prototypes are parsed from the header text, so the Python side cannot drift from
the C ABI: every function the header declares becomes an attribute with ``argtypes``
and ``restype`` set. Loading fails loudly when a shared library or a symbol is missing;
there is no fallback implementation.
"""
from __future__ import annotations

import ctypes
import re
from pathlib import Path

PKG = Path(__file__).resolve().parent
INCLUDE = PKG.parent / "include"

_SCALARS = {
    "int": ctypes.c_int,
    "int32_t": ctypes.c_int32,
    "int64_t": ctypes.c_int64,
    "uint64_t": ctypes.c_uint64,
    "size_t": ctypes.c_size_t,
    "float": ctypes.c_float,
    "double": ctypes.c_double,
    "long": ctypes.c_long,
    "mt_segment_cb": ctypes.c_void_p,  # function pointer typedef in mt_capi.h
}

_PROTO = re.compile(r"^\s*((?:const\s+)?[A-Za-z_][A-Za-z0-9_]*\s*\**)\s*\b((?:pk|mt)_[a-z0-9_]+)\s*\(([^;{]*)\)\s*;",
                    re.M | re.S)


def _strip_comments(text: str) -> str:
    text = re.sub(r"/\*.*?\*/", " ", text, flags=re.S)
    return re.sub(r"//[^\n]*", " ", text)


def _ctype(decl: str):
    decl = decl.strip()
    if decl in ("void", ""):
        return None
    if "(*" in decl:  # function pointer
        return ctypes.c_void_p
    if "*" in decl:
        base = decl.replace("const", "").split("*")[0].strip()
        if base == "char" and decl.count("*") == 1:
            return ctypes.c_char_p
        return ctypes.c_void_p
    # drop the parameter name
    parts = decl.replace("const", "").split()
    tname = parts[0] if len(parts) == 1 else " ".join(parts[:-1])
    tname = tname.strip()
    if tname in _SCALARS:
        return _SCALARS[tname]
    raise ValueError(f"unhandled C type in header: {decl!r}")


def parse_header(path: Path):
    """Returns {name: (restype, [argtypes])} for every prototype in the header."""
    text = _strip_comments(path.read_text())
    out = {}
    for m in _PROTO.finditer(text):
        ret, name, args = m.group(1).strip(), m.group(2), m.group(3)
        if ret.startswith("typedef"):
            continue
        argtypes = []
        depth = 0
        cur = ""
        pieces = []
        for ch in args:
            if ch == "(":
                depth += 1
            elif ch == ")":
                depth -= 1
            if ch == "," and depth == 0:
                pieces.append(cur)
                cur = ""
            else:
                cur += ch
        pieces.append(cur)
        for a in pieces:
            t = _ctype(a)
            if t is not None:
                argtypes.append(t)
        if "*" in ret and "char" in ret:
            restype = ctypes.c_char_p
        elif "*" in ret:
            restype = ctypes.c_void_p
        else:
            restype = _SCALARS.get(ret.replace("const", "").strip(), ctypes.c_int)
        out[name] = (restype, argtypes)
    return out


class CLib:
    """A shared library with prototypes taken from a header."""

    def __init__(self, lib_path: Path, header: Path, mode=ctypes.DEFAULT_MODE):
        if not lib_path.exists():
            raise ImportError(
                f"{lib_path} is missing: build it with `python -m paperkiln_b200.build` "
                "(the library has no CPU fallback)")
        self.path = lib_path
        self.protos = parse_header(header)
        self.dll = ctypes.CDLL(str(lib_path), mode=mode)
        for name, (restype, argtypes) in self.protos.items():
            try:
                fn = getattr(self.dll, name)
            except AttributeError as e:
                raise ImportError(f"{lib_path.name} does not export {name} declared in {header.name}") from e
            fn.restype = restype
            fn.argtypes = argtypes
            setattr(self, name, fn)


_pk = None
_mt = None


def libpk() -> CLib:
    global _pk
    if _pk is None:
        _pk = CLib(PKG / "libpk.so", INCLUDE / "pk.h", mode=ctypes.RTLD_GLOBAL)
    return _pk


def libmt() -> CLib:
    global _mt
    if _mt is None:
        libpk()
        _mt = CLib(PKG / "libmicrotorch.so", INCLUDE / "mt_capi.h")
    return _mt


class PkError(RuntimeError):
    pass


def check(rc: int, what: str = "libpk call"):
    if rc != 0:
        msg = libpk().pk_last_error().decode(errors="replace")
        raise PkError(f"{what} failed with status {rc}: {msg}")
