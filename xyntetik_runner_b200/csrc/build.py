"""Compiling the CUDA sources of this folder into one shared library for sm_100a, and the C++ sources under
host/ into a second one (see the end of this file).

The library is plain CUDA with `extern "C"` launchers (no Python or torch
headers), so a file compiles in seconds.  It is built in-tree
(`csrc/_build/libxrb200.so`) the first time it is needed, and again whenever a
source, a header or the flags change (a digest beside the library says what it
was built from).  When the tree is not writable the build goes to a per-user
folder under the system's temporary directory.  While nvcc runs, a line is
printed every few seconds.  There is no fallback: without nvcc or with a
compile error the caller gets an exception.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from typing import List

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_NAME = "libxrb200.so"
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]


# XRB200_TRACE=1: a library of its own (libxrb200_trace.so) in which every kernel's first thread writes down when
# it became resident and when the kernel ahead of it in the stream was complete (common.cuh: XR_TRACE), for
# `python -m xyntetik_runner_b200.probe timeline`.  Never the library that serves.
TRACE = os.environ.get("XRB200_TRACE", "0") not in ("", "0")
if TRACE:
    NVCC_FLAGS = NVCC_FLAGS + ["-DXR_TRACE"]
    LIB_NAME = "libxrb200_trace.so"


class BuildError(RuntimeError):
    pass


def sources() -> List[str]:
    return sorted(f for f in os.listdir(HERE) if f.endswith(".cu"))


def _headers() -> List[str]:
    return sorted(f for f in os.listdir(HERE) if f.endswith((".cuh", ".h")))


def _digest() -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    for f in sources() + _headers():
        h.update(f.encode())
        with open(os.path.join(HERE, f), "rb") as fh:
            h.update(fh.read())
    return h.hexdigest()


def find_nvcc() -> str:
    for cand in (os.environ.get("XRB200_NVCC"),
                 os.path.join(os.environ.get("CUDA_HOME", ""), "bin", "nvcc") if os.environ.get("CUDA_HOME") else None,
                 shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc not found (looked at $XRB200_NVCC, $CUDA_HOME/bin, PATH, /usr/local/cuda/bin); "
                     "the CUDA kernels cannot be built and there is no other path")


def _build_dirs() -> List[str]:
    dirs = [os.path.join(HERE, "_build")]
    tag = f"xrb200-build-{os.getuid()}"
    dirs.append(os.path.join(tempfile.gettempdir(), tag))
    return dirs


def _writable(d: str) -> bool:
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".probe-{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return True
    except OSError:
        return False


def _say(msg: str) -> None:
    print(f"[xrb200 build] {msg}", file=sys.stderr, flush=True)


def library_path(build: bool = True, verbose: bool = True) -> str:
    """Path of an up-to-date library; compiles it if needed (and allowed)."""
    digest = _digest()
    for d in _build_dirs():
        lib, stamp = os.path.join(d, LIB_NAME), os.path.join(d, "digest_trace.txt" if TRACE else "digest.txt")
        if os.path.isfile(lib) and os.path.isfile(stamp):
            with open(stamp) as f:
                if f.read().strip() == digest:
                    return lib
    if not build:
        raise BuildError("the CUDA library is not built")
    for d in _build_dirs():
        if _writable(d):
            return _compile(d, digest, verbose)
    raise BuildError("no writable folder for the build: " + ", ".join(_build_dirs()))


def _compile(out_dir: str, digest: str, verbose: bool) -> str:
    nvcc = find_nvcc()
    srcs = sources()
    t0 = time.time()
    if verbose:
        _say(f"compiling {len(srcs)} CUDA files for sm_100a into {out_dir}")
    stop = threading.Event()

    def ticker():
        while not stop.wait(5.0):
            _say(f"still compiling ... {time.time() - t0:.0f} s")
    th = threading.Thread(target=ticker, daemon=True)
    if verbose:
        th.start()
    env = dict(os.environ)
    env.setdefault("TMPDIR", out_dir)          # nvcc's intermediates; HOME may be empty or read-only

    def one(src: str) -> str:
        obj = os.path.join(out_dir, src[:-3] + f".{os.getpid()}.o")
        cmd = [nvcc] + NVCC_FLAGS + ["-I", HERE, "-c", os.path.join(HERE, src), "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True, env=env)
        if r.returncode != 0:
            raise BuildError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
        return obj
    try:
        with ThreadPoolExecutor(max_workers=min(len(srcs), os.cpu_count() or 4)) as ex:
            objs = list(ex.map(one, srcs))
        tmp_lib = os.path.join(out_dir, f".{LIB_NAME}.{os.getpid()}")
        cmd = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", tmp_lib] + objs
        r = subprocess.run(cmd, capture_output=True, text=True, env=env)
        if r.returncode != 0:
            raise BuildError(f"link failed:\n{r.stdout}\n{r.stderr}")
        lib = os.path.join(out_dir, LIB_NAME)
        os.replace(tmp_lib, lib)                      # atomic: a concurrent reader sees old or new
        with open(os.path.join(out_dir, "digest_trace.txt" if TRACE else "digest.txt"), "w") as f:
            f.write(digest + "\n")
    finally:
        stop.set()
        for src in srcs:                              # objects of this run, also of one that failed half way
            try:
                os.remove(os.path.join(out_dir, src[:-3] + f".{os.getpid()}.o"))
            except OSError:
                pass
    if verbose:
        _say(f"built {LIB_NAME} in {time.time() - t0:.1f} s")
    return lib


# ---------------------------------------------------------------------------------------------
# The host library: the C++ sources under host/ (page pools, block tables, step descriptions; no CUDA) built with
# the C++ compiler into libxrhost.so, by the same rules: in-tree, rebuilt when a source changes, no fallback.
# ---------------------------------------------------------------------------------------------
HOST_DIR = os.path.join(HERE, "host")
HOST_LIB = "libxrhost.so"
HOST_FLAGS = ["-O2", "-std=c++17", "-Wall", "-Wextra", "-shared", "-fPIC", "-fvisibility=hidden"]


def host_sources() -> List[str]:
    return sorted(f for f in os.listdir(HOST_DIR) if f.endswith(".cpp"))


def find_cxx() -> str:
    for cand in (os.environ.get("XRB200_CXX"), os.environ.get("CXX"), "g++", "c++", "clang++"):
        path = shutil.which(cand) if cand else None
        if path:
            return path
    raise BuildError("no C++ compiler found (looked at $XRB200_CXX, $CXX, g++, c++, clang++); "
                     "the host library cannot be built and there is no other path")


def host_library_path(build: bool = True) -> str:
    """Path of an up-to-date host library; compiles it if needed (and allowed)."""
    h = hashlib.sha256()
    h.update(" ".join(HOST_FLAGS).encode())
    for f in host_sources():
        h.update(f.encode())
        with open(os.path.join(HOST_DIR, f), "rb") as fh:
            h.update(fh.read())
    digest = h.hexdigest()
    for d in _build_dirs():
        lib, stamp = os.path.join(d, HOST_LIB), os.path.join(d, "digest_host.txt")
        if os.path.isfile(lib) and os.path.isfile(stamp):
            with open(stamp) as f:
                if f.read().strip() == digest:
                    return lib
    if not build:
        raise BuildError("the host library is not built")
    for d in _build_dirs():
        if not _writable(d):
            continue
        tmp_lib = os.path.join(d, f".{HOST_LIB}.{os.getpid()}")
        cmd = [find_cxx()] + HOST_FLAGS + ["-o", tmp_lib] + [os.path.join(HOST_DIR, f) for f in host_sources()]
        env = dict(os.environ)
        env.setdefault("TMPDIR", d)
        r = subprocess.run(cmd, capture_output=True, text=True, env=env)
        if r.returncode != 0:
            raise BuildError(f"the C++ compiler failed on the host library:\n{r.stdout}\n{r.stderr}")
        lib = os.path.join(d, HOST_LIB)
        os.replace(tmp_lib, lib)
        with open(os.path.join(d, "digest_host.txt"), "w") as f:
            f.write(digest + "\n")
        return lib
    raise BuildError("no writable folder for the build: " + ", ".join(_build_dirs()))


if __name__ == "__main__":
    print(library_path())
    print(host_library_path())
