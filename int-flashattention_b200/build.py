"""Build step for libintfa.so: one nvcc invocation over csrc/*.cu for sm_100a.

The library is built IN-TREE (next to this file) so that it travels with the
source tree; it is never installed into site-packages.
"""
import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
LIB = os.path.join(PKG_DIR, "libintfa.so")
SOURCES = ["intfa_api.cu", "intfa_quant.cu", "intfa_fwd.cu"]
HEADERS = ["intfa_internal.h", "intfa_ptx.cuh", "intfa_fwd_pipe.cuh", "intfa_fwd_pipe_softmax.inc",
           "intfa_fwd_pipe_update.inc", os.path.join("..", "..", "include", "intfa.h")]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-shared", "-Xcompiler", "-fPIC"]


def _stale():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in SOURCES + HEADERS]
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def build(force=False, verbose=False):
    """Compile csrc/ into libintfa.so if it is missing or older than its sources."""
    if not force and not _stale():
        return LIB
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-o", LIB] + SOURCES
    res = subprocess.run(cmd, cwd=CSRC, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed building libintfa.so (exit %d)" % res.returncode)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
