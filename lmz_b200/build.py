"""Build the CUDA library in-tree with nvcc for sm_100a.

The counterpart of the reference's build-on-first-use step
(lmz/gpu/build.py:168-274), simplified: one fixed architecture, no driver
probing, and the artifact sits beside its sources so it travels with the tree.
"""
from __future__ import annotations

import contextlib
import fcntl
import os
import shutil
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(CSRC, "liblmz_b200.so")
SOURCES = ["lmz_b200.cu"]
last_error = ""

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "--extended-lambda", "-shared", "-Xcompiler", "-fPIC"]


def find_nvcc() -> str | None:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    return cand if cand and os.path.exists(cand) else None


def _stale() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cu", ".cuh", ".inl"))]
    deps.append(os.path.join(os.path.dirname(HERE), "include", "lmz_b200.h"))
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


@contextlib.contextmanager
def _build_lock():
    """An exclusive lock on a file beside the library (no lock where the directory is
    read-only: the compile then fails on its own account)."""
    try:
        f = open(LIB + ".lock", "w")
    except OSError:
        yield
        return
    try:
        fcntl.flock(f, fcntl.LOCK_EX)
        yield
    finally:
        f.close()


def build(force: bool = False, verbose: bool = False) -> str | None:
    """Path of the built library, compiling it if sources are newer. None on failure
    (reason in `last_error`); never raises."""
    global last_error
    prebuilt = os.environ.get("LMZ_B200_LIBRARY")
    if prebuilt:                       # a library built elsewhere (deployment without nvcc)
        if os.path.exists(prebuilt):
            return prebuilt
        last_error = f"LMZ_B200_LIBRARY names a missing file: {prebuilt}"
        return None
    if not force and not _stale():
        return LIB
    nvcc = find_nvcc()
    if nvcc is None:
        if os.path.exists(LIB):
            return LIB
        last_error = "nvcc was not found (set NVCC or put it on PATH)"
        return None
    # Several processes may get here at once (one rank per GPU): one of them compiles, the
    # others wait on the lock and find the library fresh; each output file has its own name,
    # and the rename is atomic.
    with _build_lock():
        if not force and not _stale():
            return LIB
        tmp = f"{LIB}.{os.getpid()}.tmp"
        cmd = [nvcc, *NVCC_FLAGS, "-o", tmp, *SOURCES]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        try:
            p = subprocess.run(cmd, cwd=CSRC, capture_output=True, text=True, timeout=900)
        except Exception as exc:
            last_error = f"nvcc did not run: {exc}"
            return None
        if verbose:
            print(p.stderr)
        if p.returncode != 0:
            last_error = "nvcc failed: " + (p.stderr.strip().splitlines() or ["?"])[-1]
            if os.path.exists(tmp):
                os.unlink(tmp)
            return None
        os.replace(tmp, LIB)
        return LIB


if __name__ == "__main__":
    print(build(force=True, verbose=True) or last_error)
