"""Builds the engine's native libraries in-tree, at first use.

* ``libxinfer_b200_kernels.so``: every ``.cu`` file of this folder, compiled by nvcc for sm_100a.
* ``libxinfer_b200_host.so``: the host runtime (``host/*.cpp``: page pools, block tables, request
  slots, scheduler), compiled by g++; it needs no CUDA and also serves the CPU-only tests.

Both land in ``csrc/_build`` next to a stamp of the sources' hash, so a changed source rebuilds
and an unchanged one loads at once.  A line is printed now and then while compiling.
"""
from __future__ import annotations

import concurrent.futures
import hashlib
import os
import shutil
import subprocess
import sys
import time
from typing import List, Sequence

_HERE = os.path.dirname(os.path.abspath(__file__))
BUILD_DIR = os.path.join(_HERE, "_build")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-Wall"]


class BuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[xinfer_b200 build] {msg}", file=sys.stderr, flush=True)


def _find_nvcc() -> str:
    for cand in (os.environ.get("XINFER_B200_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc was not found (PATH, /usr/local/cuda/bin): the CUDA kernels cannot be compiled, "
                     "and this engine has no other way to run")


def _sources(sub: str, ext: str) -> List[str]:
    d = os.path.join(_HERE, sub) if sub else _HERE
    return sorted(os.path.join(d, f) for f in os.listdir(d) if f.endswith(ext))


def _headers() -> List[str]:
    out = _sources("", ".cuh") + _sources("", ".h")
    hd = os.path.join(_HERE, "host")
    if os.path.isdir(hd):
        out += sorted(os.path.join(hd, f) for f in os.listdir(hd) if f.endswith((".h", ".hpp")))
    return out


def _digest(files: Sequence[str], flags: Sequence[str]) -> str:
    h = hashlib.sha256()
    for f in files:
        h.update(os.path.basename(f).encode())
        with open(f, "rb") as fh:
            h.update(fh.read())
    h.update(" ".join(flags).encode())
    return h.hexdigest()


def _run(cmd: Sequence[str], what: str) -> None:
    t0 = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    while True:
        try:
            out, _ = proc.communicate(timeout=20)
            break
        except subprocess.TimeoutExpired:
            _say(f"still compiling {what} ({int(time.time() - t0)} s)")
    if proc.returncode != 0:
        raise BuildError(f"compiling {what} failed:\n{' '.join(cmd)}\n{out}")
    if out.strip() and os.environ.get("XINFER_B200_BUILD_VERBOSE"):
        _say(out.strip())


def _up_to_date(lib: str, stamp: str, digest: str) -> bool:
    if not (os.path.isfile(lib) and os.path.isfile(stamp)):
        return False
    with open(stamp, "r") as f:
        return f.read().strip() == digest


def _build(lib_name: str, sources: List[str], compiler_cmd, link_cmd, flags, what: str) -> str:
    os.makedirs(BUILD_DIR, exist_ok=True)
    lib = os.path.join(BUILD_DIR, lib_name)
    stamp = lib + ".stamp"
    digest = _digest(sources + _headers(), flags)
    if _up_to_date(lib, stamp, digest):
        return lib
    _say(f"compiling {what}: {len(sources)} file(s), this happens once")
    t0 = time.time()
    objs = []
    jobs = []
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(sources))) as pool:
        for src in sources:
            obj = os.path.join(BUILD_DIR, os.path.splitext(os.path.basename(src))[0] + f".{os.getpid()}.o")
            objs.append(obj)
            jobs.append(pool.submit(_run, compiler_cmd(src, obj), os.path.basename(src)))
        for j in jobs:
            j.result()
    tmp = lib + f".{os.getpid()}.tmp"
    _run(link_cmd(objs, tmp), lib_name)
    os.replace(tmp, lib)
    for o in objs:
        try:
            os.remove(o)
        except OSError:
            pass
    with open(stamp, "w") as f:
        f.write(digest)
    _say(f"{lib_name} ready in {time.time() - t0:.0f} s")
    return lib


def build_kernels() -> str:
    nvcc = None
    sources = _sources("", ".cu")
    flags = list(NVCC_FLAGS)

    def cc(src, obj):
        return [nvcc or _find_nvcc(), *flags, "-I", _HERE, "-c", src, "-o", obj]

    def ld(objs, out):
        return [nvcc or _find_nvcc(), "-shared", "-o", out, *objs, "-lcuda"]

    return _build("libxinfer_b200_kernels.so", sources, cc, ld, flags, "CUDA kernels for sm_100a")


def build_host() -> str:
    cxx = shutil.which("g++") or shutil.which("c++")
    if not cxx:
        raise BuildError("no C++ compiler (g++) found: the host runtime cannot be compiled")
    sources = _sources("host", ".cpp")
    flags = list(CXX_FLAGS)

    def cc(src, obj):
        return [cxx, *flags, "-I", os.path.join(_HERE, "host"), "-c", src, "-o", obj]

    def ld(objs, out):
        return [cxx, "-shared", "-o", out, *objs]

    return _build("libxinfer_b200_host.so", sources, cc, ld, flags, "host runtime")


def build_all() -> None:
    build_host()
    build_kernels()


if __name__ == "__main__":
    build_all()
