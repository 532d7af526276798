"""Builds the CUDA library of this package for sm_100a and finds the built file.

The sources under ``csrc/`` are plain CUDA with an ``extern "C"`` interface (no PyTorch headers),
so each file compiles in seconds.  The library is built in-tree (``csrc/_build/``) at first use
and rebuilt when a source changes (a digest of the sources and flags is stored beside it); a
source tree that is not writable builds into a per-user folder under the temporary directory.
While it compiles it prints a line per file so that a first call in a fresh checkout is not silent.
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
from typing import List, Optional

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")
LIB_NAME = "libpe_b200.so"
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


class BuildError(RuntimeError):
    pass


def _find_nvcc() -> str:
    for cand in (os.environ.get("PE_B200_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError(
        "nvcc was not found (looked at $PE_B200_NVCC, PATH and /usr/local/cuda/bin): the CUDA kernels of "
        "this package cannot be built, and there is no fallback without them"
    )


def sources() -> List[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _headers() -> List[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h")))


def digest() -> str:
    h = hashlib.sha256()
    for path in sources() + _headers():
        h.update(os.path.basename(path).encode())
        with open(path, "rb") as fh:
            h.update(fh.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()[:24]


def _build_dirs() -> List[str]:
    dirs = [os.path.join(CSRC, "_build")]
    uid = os.getuid() if hasattr(os, "getuid") else 0
    dirs.append(os.path.join(tempfile.gettempdir(), f"pe_b200_build_{uid}"))
    return dirs


def _is_current(build_dir: str, want: str) -> bool:
    lib = os.path.join(build_dir, LIB_NAME)
    stamp = os.path.join(build_dir, "digest.txt")
    if not (os.path.isfile(lib) and os.path.isfile(stamp)):
        return False
    with open(stamp) as fh:
        return fh.read().strip() == want


def find_built() -> Optional[str]:
    want = digest()
    for d in _build_dirs():
        if _is_current(d, want):
            return os.path.join(d, LIB_NAME)
    return None


def _say(msg: str) -> None:
    print(f"[pytorch-engine_b200] {msg}", file=sys.stderr, flush=True)


def build(verbose: bool = True, force: bool = False) -> str:
    """Compile every ``csrc/*.cu`` for sm_100a and link ``libpe_b200.so``; returns its path."""
    want = digest()
    if not force:
        lib = find_built()
        if lib:
            return lib
    nvcc = _find_nvcc()
    build_dir = None
    for d in _build_dirs():
        try:
            os.makedirs(d, exist_ok=True)
            probe = os.path.join(d, f".w{os.getpid()}")
            with open(probe, "w"):
                pass
            os.remove(probe)
            build_dir = d
            break
        except OSError:
            continue
    if build_dir is None:
        raise BuildError(f"no writable build folder among {_build_dirs()}")
    srcs = sources()
    if verbose:
        _say(f"compiling {len(srcs)} CUDA files for sm_100a into {build_dir} (first use, or a source changed)")
    t0 = time.time()
    done = threading.Event()

    def _ticker():
        while not done.wait(10.0):
            if verbose:
                _say(f"... still compiling ({time.time() - t0:.0f} s)")

    tick = threading.Thread(target=_ticker, daemon=True)
    tick.start()

    def _compile(src: str) -> str:
        obj = os.path.join(build_dir, os.path.basename(src)[:-3] + f".{os.getpid()}.o")
        cmd = [nvcc, *NVCC_FLAGS, "-I", CSRC, "-c", src, "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise BuildError(f"nvcc failed on {os.path.basename(src)}:\n{r.stdout}\n{r.stderr}")
        if verbose:
            _say(f"compiled {os.path.basename(src)} ({time.time() - t0:.0f} s)")
        return obj

    try:
        with ThreadPoolExecutor(max_workers=min(8, max(1, os.cpu_count() or 1))) as ex:
            objs = list(ex.map(_compile, srcs))
        tmp_lib = os.path.join(build_dir, f"{LIB_NAME}.{os.getpid()}.tmp")
        cmd = [nvcc, "-shared", "-o", tmp_lib, *objs, "-gencode", "arch=compute_100a,code=sm_100a"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise BuildError(f"linking {LIB_NAME} failed:\n{r.stdout}\n{r.stderr}")
        os.replace(tmp_lib, os.path.join(build_dir, LIB_NAME))
        with open(os.path.join(build_dir, "digest.txt"), "w") as fh:
            fh.write(want + "\n")
        for o in objs:
            try:
                os.remove(o)
            except OSError:
                pass
    finally:
        done.set()
    if verbose:
        _say(f"built {LIB_NAME} in {time.time() - t0:.0f} s")
    return os.path.join(build_dir, LIB_NAME)
