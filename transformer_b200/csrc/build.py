"""Compile the CUDA sources of this folder for sm_100a into one shared library.

The library is built at its first use: ``nvcc`` per source file (in parallel), then one link.  The
result is keyed by a hash of the sources and flags, so an edited source is rebuilt and an old
library is never loaded by mistake.  It lands in ``_build/`` beside the sources when that folder can
be written, else in a per-user folder under the system's temporary directory; HOME is never used.
While it compiles it prints a line now and then to stderr.

There is no fallback: a missing compiler or a failed build raises :class:`KernelBuildError`.
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
LIB_NAME = "libtransformer_b200.so"
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


class KernelBuildError(RuntimeError):
    pass


def sources() -> List[str]:
    return sorted(f for f in os.listdir(HERE) if f.endswith(".cu"))


def _headers() -> List[str]:
    return sorted(f for f in os.listdir(HERE) if f.endswith((".cuh", ".h")))


def find_nvcc() -> str:
    cands = []
    for env in ("CUDA_HOME", "CUDA_PATH"):
        if os.environ.get(env):
            cands.append(os.path.join(os.environ[env], "bin", "nvcc"))
    cands.append("/usr/local/cuda/bin/nvcc")
    w = shutil.which("nvcc")
    if w:
        cands.append(w)
    for c in cands:
        if os.path.isfile(c) and os.access(c, os.X_OK):
            return c
    raise KernelBuildError("nvcc not found (looked in $CUDA_HOME/bin, /usr/local/cuda/bin and PATH); "
                           "the CUDA kernels of transformer_b200 cannot be built and there is no fallback")


def source_hash() -> str:
    h = hashlib.sha256()
    for f in sources() + _headers():
        h.update(f.encode())
        with open(os.path.join(HERE, f), "rb") as fh:
            h.update(fh.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()[:16]


def _writable_dir(path: str) -> bool:
    try:
        os.makedirs(path, exist_ok=True)
        probe = os.path.join(path, f".probe-{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return True
    except OSError:
        return False


def build_dir() -> str:
    key = source_hash()
    in_tree = os.path.join(HERE, "_build", key)
    if os.path.isfile(os.path.join(in_tree, LIB_NAME)) or _writable_dir(in_tree):
        return in_tree
    tmp = os.path.join(tempfile.gettempdir(), f"transformer_b200-{os.getuid()}", key)
    if _writable_dir(tmp):
        return tmp
    raise KernelBuildError(f"neither {in_tree} nor {tmp} can be written; nowhere to build the kernels")


def _say(msg: str) -> None:
    print(f"[transformer_b200] {msg}", file=sys.stderr, flush=True)


def _compile_one(nvcc: str, src: str, out_dir: str) -> str:
    obj = os.path.join(out_dir, src[:-3] + ".o")
    cmd = [nvcc, *NVCC_FLAGS, "-I", HERE, "-c", os.path.join(HERE, src), "-o", obj]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise KernelBuildError(f"nvcc failed on {src}:\n{r.stdout}")
    return obj


def ensure_built(verbose: bool = True) -> str:
    """Path of the shared library, building it first if it is not there."""
    out_dir = build_dir()
    lib = os.path.join(out_dir, LIB_NAME)
    if os.path.isfile(lib):
        return lib
    nvcc = find_nvcc()
    srcs = sources()
    if verbose:
        _say(f"compiling {len(srcs)} CUDA files for sm_100a into {out_dir} (first use only)")
    t0 = time.time()
    done = threading.Event()

    def ticker():
        while not done.wait(10.0):
            _say(f"still compiling ... {time.time() - t0:.0f} s")

    th = threading.Thread(target=ticker, daemon=True)
    if verbose:
        th.start()
    try:
        with ThreadPoolExecutor(max_workers=min(len(srcs), os.cpu_count() or 4)) as pool:
            objs = list(pool.map(lambda s: _compile_one(nvcc, s, out_dir), srcs))
        tmp_lib = lib + f".{os.getpid()}.tmp"
        r = subprocess.run([nvcc, "-shared", "-o", tmp_lib, *objs],
                           stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if r.returncode != 0:
            raise KernelBuildError(f"link failed:\n{r.stdout}")
        os.replace(tmp_lib, lib)   # atomic: a concurrent process sees the old state or the whole file
        for o in objs:
            try:
                os.remove(o)
            except OSError:
                pass
    finally:
        done.set()
    _prune(os.path.dirname(out_dir), keep=os.path.basename(out_dir))
    if verbose:
        _say(f"built {LIB_NAME} in {time.time() - t0:.0f} s")
    return lib


def _prune(parent: str, keep: str) -> None:
    """Libraries of earlier states of the sources are of no use once the present one is built."""
    try:
        for name in os.listdir(parent):
            old = os.path.join(parent, name)
            if name != keep and len(name) == len(keep) and os.path.isfile(os.path.join(old, LIB_NAME)):
                shutil.rmtree(old, ignore_errors=True)
    except OSError:
        pass


if __name__ == "__main__":
    print(ensure_built())
