"""Compile the CUDA sources into the in-tree shared library (plain nvcc, sm_100a only)."""

import os
import shutil
import subprocess

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
INCLUDE = os.path.join(os.path.dirname(PKG_DIR), "include")
LIB_PATH = os.path.join(CSRC, "libpylo_b200.so")
LOCK_PATH = os.path.join(CSRC, ".build.lock")
SOURCES = [os.path.join(CSRC, "pylo_kernels.cu")]
HEADERS = [os.path.join(CSRC, "pylo_common.cuh"), os.path.join(CSRC, "pylo_apply_tc.cuh"), os.path.join(CSRC, "pylo_ns_gemm.cuh"), os.path.join(INCLUDE, "pylo_b200.h")]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC", "-shared",
]


def find_nvcc():
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    return cand if os.path.exists(cand) else None


def is_stale():
    if not os.path.exists(LIB_PATH):
        return True
    built = os.path.getmtime(LIB_PATH)
    return any(os.path.getmtime(f) > built for f in SOURCES + HEADERS if os.path.exists(f))


def build(force=False, verbose=False):
    """Build ``csrc/libpylo_b200.so``; returns its path.  Raises if nvcc is missing or fails.

    Safe to call from several processes at once (one rank per GPU importing the package): a file lock lets one of
    them compile, into a temporary file that is renamed over the library in one step, while the others wait and
    then find the library up to date."""
    if not force and not is_stale():
        return LIB_PATH
    nvcc = find_nvcc()
    if nvcc is None:
        raise RuntimeError("nvcc not found: cannot build pylo_b200/csrc/libpylo_b200.so")
    import fcntl

    with open(LOCK_PATH, "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if not force and not is_stale():   # another process built it while this one waited
                return LIB_PATH
            # PYLO_B200_NVCC_FLAGS: extra nvcc flags for a one-off build (e.g. -DTC_STAGE_CLOCKS for the stage
            # clocks of the tensor-core apply kernel)
            extra = os.environ.get("PYLO_B200_NVCC_FLAGS", "").split()
            tmp = f"{LIB_PATH}.tmp.{os.getpid()}"
            cmd = [nvcc] + NVCC_FLAGS + extra + ["-I", INCLUDE, "-I", CSRC, "-o", tmp] + SOURCES
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            res = subprocess.run(cmd, capture_output=True, text=True)
            if res.returncode != 0:
                if os.path.exists(tmp):
                    os.remove(tmp)
                raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
            os.replace(tmp, LIB_PATH)
            if verbose:
                print(res.stderr)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
    return LIB_PATH


if __name__ == "__main__":
    import sys

    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
