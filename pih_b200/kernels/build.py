"""Builds the kernel pack: ``csrc/*.cu`` -> one shared library for sm_100a.

The library is plain ``extern "C"`` entry points over raw device pointers, so
it needs neither torch's headers nor its ABI: nvcc compiles each ``.cu`` in
seconds and the result loads through ``ctypes``.  It is built in-tree (next
to this file) when the tree is writable, else under the system's temporary
folder; a stamp of the sources' hash decides whether a rebuild is needed.
Progress is printed to stderr while it compiles.
"""
from __future__ import annotations

import concurrent.futures
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time
from typing import List

_HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.normpath(os.path.join(_HERE, "..", "csrc"))
LIB_NAME = "libpih_b200_kernels.so"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]


def _nvcc() -> str:
    for cand in (os.environ.get("PIH_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("pih_b200: nvcc was not found (set PIH_NVCC); the kernel pack cannot be built")


def sources() -> List[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _source_hash() -> str:
    h = hashlib.sha256()
    for f in sorted(os.listdir(CSRC)):
        if f.endswith((".cu", ".cuh", ".h")):
            h.update(f.encode())
            with open(os.path.join(CSRC, f), "rb") as fh:
                h.update(fh.read())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
    return h.hexdigest()[:16]


def _build_dir() -> str:
    in_tree = os.path.join(_HERE, "_build")
    try:
        os.makedirs(in_tree, exist_ok=True)
        probe = os.path.join(in_tree, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return in_tree
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"pih_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def _say(msg: str) -> None:
    print(f"[pih_b200 build] {msg}", file=sys.stderr, flush=True)


def _compile_one(nvcc: str, src: str, obj: str) -> None:
    cmd = [nvcc] + ARCH_FLAGS + NVCC_FLAGS + ["-I", CSRC, "-c", src, "-o", obj]
    t0 = time.time()
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"pih_b200: nvcc failed on {os.path.basename(src)}:\n{proc.stdout}")
    _say(f"compiled {os.path.basename(src)} in {time.time() - t0:.1f} s")


def library_path(build: bool = True) -> str:
    """Path of the built library; builds it first when it is missing or stale."""
    bdir = _build_dir()
    lib = os.path.join(bdir, LIB_NAME)
    stamp = os.path.join(bdir, "stamp.txt")
    want = _source_hash()
    if os.path.exists(lib) and os.path.exists(stamp):
        with open(stamp) as f:
            if f.read().strip() == want:
                return lib
    if not build:
        raise RuntimeError(f"pih_b200: {lib} is missing or stale")
    nvcc = _nvcc()
    srcs = sources()
    _say(f"compiling {len(srcs)} CUDA sources for sm_100a into {bdir} (first call only)")
    t0 = time.time()
    objs = [os.path.join(bdir, os.path.basename(s)[:-3] + ".o") for s in srcs]
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as pool:
        futures = [pool.submit(_compile_one, nvcc, s, o) for s, o in zip(srcs, objs)]
        pending = set(futures)
        while pending:
            done, pending = concurrent.futures.wait(pending, timeout=15)
            for d in done:
                d.result()
            if pending:
                _say(f"still compiling ({len(pending)} of {len(srcs)} left, {time.time() - t0:.0f} s)")
    tmp = lib + f".tmp{os.getpid()}"
    cmd = [nvcc] + ARCH_FLAGS + ["-shared", "-o", tmp] + objs
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"pih_b200: linking the kernel pack failed:\n{proc.stdout}")
    os.replace(tmp, lib)
    with open(stamp, "w") as f:
        f.write(want)
    _say(f"built {LIB_NAME} in {time.time() - t0:.1f} s")
    return lib
