"""In-tree build of the two shared libraries of this package.

  libpk.so            CUDA kernels for sm_100a behind the C ABI of include/pk.h
  libmicrotorch.so    C++ host library: the microtorch tape, ops, layers, models and
                      the C driver entry points of include/mt_capi.h; calls libpk.so
                      through the C ABI only

Both are written next to this file so that they travel with the source tree.
Run as a script (``python -m paperkiln_b200.build``) or call :func:`build_all`.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
HOST = PKG / "host"
INCLUDE = ROOT / "include"
OBJ = PKG / "build"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
    "-I", str(INCLUDE), "-I", str(CSRC),
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found; libpk.so cannot be built")


def _host_cxx() -> str:
    # The environment's CXX may point at a compiler without the libraries nvcc expects.
    for cand in ("/usr/bin/g++", shutil.which("g++")):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("g++ not found")


def _newer(target: Path, sources) -> bool:
    if not target.exists():
        return False
    t = target.stat().st_mtime
    return all(Path(s).stat().st_mtime <= t for s in sources)


def _run(cmd, verbose):
    if verbose:
        print(" ".join(str(c) for c in cmd), flush=True)
    res = subprocess.run([str(c) for c in cmd], capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError(f"build step failed: {' '.join(str(c) for c in cmd[:3])} ...")
    if verbose and (res.stdout or res.stderr):
        print(res.stdout + res.stderr, flush=True)


def build_libpk(verbose: bool = False, force: bool = False, ptxas_info: bool = False) -> Path:
    OBJ.mkdir(exist_ok=True)
    nvcc = _nvcc()
    cxx = _host_cxx()
    headers = list(CSRC.glob("*.cuh")) + list(INCLUDE.glob("*.h"))
    objs, jobs = [], []
    for src in sorted(CSRC.glob("*.cu")):
        obj = OBJ / (src.stem + ".o")
        if force or not _newer(obj, [src, *headers]):
            cmd = [nvcc, "-ccbin", cxx, *NVCC_FLAGS, *os.environ.get("PK_NVCC_EXTRA", "").split(), "-c", src, "-o", obj]
            if ptxas_info:
                cmd[1:1] = ["-Xptxas", "-v"]
            jobs.append(cmd)
        objs.append(obj)
    if jobs:  # translation units are independent: compile them side by side
        from concurrent.futures import ThreadPoolExecutor
        with ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 4)) as pool:
            list(pool.map(lambda c: _run(c, verbose or ptxas_info), jobs))
    lib = PKG / "libpk.so"
    if force or not _newer(lib, objs):
        # cudart is linked statically (nvcc default) and the driver API is reached through
        # cudaGetDriverEntryPoint, so the library loads on a machine without a GPU driver.
        _run([nvcc, "-ccbin", cxx, "-shared", "-o", lib, *objs], verbose)
    return lib


def build_host(verbose: bool = False, force: bool = False) -> Path:
    OBJ.mkdir(exist_ok=True)
    cxx = _host_cxx()
    headers = list((HOST / "include" / "microtorch").glob("*.hpp")) + list(INCLUDE.glob("*.h"))
    flags = ["-O2", "-std=c++17", "-fPIC", "-Wall", "-Wno-unused-function",
             "-I", HOST / "include", "-I", INCLUDE]
    objs = []
    for src in sorted((HOST / "src").glob("*.cpp")):
        obj = OBJ / ("host_" + src.stem + ".o")
        if force or not _newer(obj, [src, *headers]):
            _run([cxx, *flags, "-c", src, "-o", obj], verbose)
        objs.append(obj)
    lib = PKG / "libmicrotorch.so"
    if force or not _newer(lib, objs + [PKG / "libpk.so"]):
        _run([cxx, "-shared", "-o", lib, *objs, "-L", PKG, "-lpk", "-Wl,-rpath,$ORIGIN"], verbose)
    # example programs over the C driver ABI (one executable per file of host/examples)
    for src in sorted((HOST / "examples").glob("*.cpp")):
        exe = PKG / src.stem
        if force or not _newer(exe, [src, lib, *headers]):
            _run([cxx, "-O2", "-std=c++17", "-I", INCLUDE, "-I", HOST / "include", src, "-o", exe, "-L", PKG, "-lmicrotorch",
                  "-lpk", "-pthread", "-Wl,-rpath,$ORIGIN"], verbose)
    return lib


def build_all(verbose: bool = False, force: bool = False):
    return build_libpk(verbose, force), build_host(verbose, force)


if __name__ == "__main__":
    build_all(verbose="-v" in sys.argv, force="-f" in sys.argv)
    print("built", PKG / "libpk.so", PKG / "libmicrotorch.so")
