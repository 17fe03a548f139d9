"""Builds the sm_100a kernel library with nvcc and loads it through ctypes.

The library is one shared object made of the ``.cu`` files beside this file.
It is built on first use into ``_build/`` beside the sources (or, when that
folder cannot be written, into a per-user folder under the system's temporary
directory) and is named after a hash of the sources and flags, so a stale
build is never loaded.  While nvcc runs, a line is printed to stderr now and
then.  There is no fallback: if the library cannot be built or loaded the
import fails with the compiler's output.
"""
from __future__ import annotations

import concurrent.futures
import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from typing import List, Optional

HERE = os.path.dirname(os.path.abspath(__file__))
SOURCES = ["elementwise.cu", "attention.cu", "attention_mma.cu", "attention_mma_prefill.cu",
           "attention_mma_fused.cu", "attention_mma_two_warps.cu", "attention_tc.cu", "gemm_simt.cu", "gemm_tcgen05.cu", "sampling.cu"]
HEADERS = ["api.h", "common.cuh", "attention_mma.cuh", "no_alloc.h"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default"]

_lib: Optional[ctypes.CDLL] = None
_lock = threading.Lock()


class BuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[yalm_b200] {msg}", file=sys.stderr, flush=True)


def _nvcc() -> str:
    for cand in (os.environ.get("YALM_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand):
            return cand
    raise BuildError("nvcc was not found (looked at $YALM_NVCC, PATH and /usr/local/cuda/bin); "
                     "the sm_100a kernels cannot be built and there is no fallback")


def _source_hash() -> str:
    h = hashlib.sha1()
    for name in SOURCES + HEADERS:
        with open(os.path.join(HERE, name), "rb") as f:
            h.update(name.encode())
            h.update(f.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()[:16]


def _build_dir() -> str:
    d = os.path.join(HERE, "_build")
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return d
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"yalm_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def library_path() -> str:
    return os.path.join(_build_dir(), f"libyalm_b200_{_source_hash()}.so")


def _compile_one(nvcc: str, src: str, obj: str, extra: List[str]) -> None:
    cmd = [nvcc, *NVCC_FLAGS, *extra, "-I", HERE, "-c", os.path.join(HERE, src), "-o", obj]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise BuildError(f"nvcc failed on {src}:\n{' '.join(cmd)}\n{r.stdout}")
    if extra and r.stdout.strip():
        _say(r.stdout.strip())


def build(verbose_ptxas: bool = False, force: bool = False) -> str:
    """Compiles (if needed) and returns the path of the shared object."""
    path = library_path()
    if os.path.isfile(path) and not force:
        return path
    nvcc = _nvcc()
    out_dir = os.path.dirname(path)
    tag = os.path.basename(path)[len("libyalm_b200_"):-3]
    extra = ["-Xptxas", "-v"] if verbose_ptxas else []
    _say(f"building the sm_100a kernel library ({len(SOURCES)} files) into {out_dir}")
    t0 = time.time()
    objs = [os.path.join(out_dir, f"{os.path.splitext(s)[0]}_{tag}_{os.getpid()}.o") for s in SOURCES]
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(10, len(SOURCES))) as pool:
        futs = {pool.submit(_compile_one, nvcc, s, o, extra): s for s, o in zip(SOURCES, objs)}
        pending = set(futs)
        while pending:
            done, pending = concurrent.futures.wait(pending, timeout=10.0)
            for f in done:
                f.result()
                _say(f"compiled {futs[f]} ({time.time() - t0:.0f} s)")
            if pending:
                _say(f"still compiling {sorted(futs[f] for f in pending)} ({time.time() - t0:.0f} s)")
    tmp = path + f".{os.getpid()}.tmp"
    cmd = [nvcc, "-shared", "-o", tmp, *objs, "-gencode", "arch=compute_100a,code=sm_100a"]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise BuildError(f"linking failed:\n{' '.join(cmd)}\n{r.stdout}")
    os.replace(tmp, path)
    for name in os.listdir(out_dir):           # older builds of other source states
        if name.startswith("libyalm_b200_") and name.endswith(".so") and \
                os.path.join(out_dir, name) != path:
            try:
                os.remove(os.path.join(out_dir, name))
            except OSError:
                pass
    for o in objs:
        try:
            os.remove(o)
        except OSError:
            pass
    _say(f"built {os.path.basename(path)} in {time.time() - t0:.0f} s")
    return path


def load() -> ctypes.CDLL:
    """The loaded library (built first if needed)."""
    global _lib
    with _lock:
        if _lib is None:
            path = build()
            try:
                _lib = ctypes.CDLL(path)
            except OSError as e:
                raise BuildError(f"could not load {path}: {e}") from None
        return _lib
