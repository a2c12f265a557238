"""Builds libesep_head.so in-tree with nvcc for sm_100a (cross-compiles without a GPU).

    python -m esep_soup_kernels_b200.csrc.build [--force] [--verbose]
"""

import os
import shutil
import subprocess
import sys

CSRC = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(CSRC, "libesep_head.so")
SOURCES = ["esep_head.cu"]
# every header of this directory is a dependency of the one translation unit
HEADERS = sorted(f for f in os.listdir(CSRC) if f.endswith(".cuh")) + [
    os.path.join("..", "..", "include", "esep_head.h")]


def _nvcc():
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: the CUDA extension cannot be built")
    return exe


def have_nvcc():
    return bool(shutil.which("nvcc")) or os.path.exists("/usr/local/cuda/bin/nvcc")


def is_stale():
    if not os.path.exists(LIB_PATH):
        return True
    built = os.path.getmtime(LIB_PATH)
    deps = [os.path.join(CSRC, f) for f in SOURCES + HEADERS]
    return any(os.path.getmtime(d) > built for d in deps if os.path.exists(d))


def build(force=False, verbose=False):
    """Compiles the library if it is missing or older than its sources. Returns its path.

    Several processes may get here at once (the ranks of a multi-GPU job importing the package):
    the build runs under an exclusive file lock, writes to a temporary file and renames it into
    place, and whoever gets the lock second finds the library fresh and returns."""
    if not force and not is_stale():
        return LIB_PATH
    import fcntl

    with open(os.path.join(CSRC, ".build.lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        if not force and not is_stale():
            return LIB_PATH
        tmp = LIB_PATH + ".tmp.%d" % os.getpid()
        cmd = [
            _nvcc(), "-std=c++17", "-O3", "-lineinfo",
            "-gencode", "arch=compute_100a,code=sm_100a",
            "-shared", "-Xcompiler", "-fPIC",
            "-Xptxas", "-v" if verbose else "-warn-spills",
            "-o", tmp,
        ] + [os.path.join(CSRC, s) for s in SOURCES]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or res.returncode != 0:
            sys.stderr.write(res.stdout + res.stderr)
        if res.returncode != 0:
            if os.path.exists(tmp):
                os.remove(tmp)
            raise RuntimeError("nvcc failed building libesep_head.so")
        os.replace(tmp, LIB_PATH)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
