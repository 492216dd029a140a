"""Builds libheron_b200.so in-tree with nvcc for sm_100a.

    python -m heron_b200.build [--force] [--verbose]

The library is the package's only compute path.  nvcc cross-compiles without a GPU.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
TARGET = os.path.join(HERE, "libheron_b200.so")
SOURCES = [os.path.join(CSRC, "hb_api.cu")]
HEADER = os.path.join(HERE, os.pardir, "include", "heron_b200.h")


def deps():
    """Everything the one translation unit includes: all of csrc/ and the public header."""
    return [os.path.join(CSRC, f) for f in sorted(os.listdir(CSRC)) if f.endswith((".cu", ".cuh"))] + [HEADER]


NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC", "-cudart", "static",
]


def nvcc():
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.sep not in cand or os.path.exists(cand)):
            return cand
    return "nvcc"


def is_stale():
    if not os.path.exists(TARGET):
        return True
    t = os.path.getmtime(TARGET)
    return any(os.path.exists(d) and os.path.getmtime(d) > t for d in deps())


def build(force=False, verbose=False, extra_flags=()):
    """Diagnostic probe modes (knob ``probe``) are compiled in only when HB_PROBES=1 is set in the
    environment; the shipped library has none of their branches."""
    if not force and not is_stale():
        return TARGET
    if os.environ.get("HB_PROBES") == "1":
        extra_flags = list(extra_flags) + ["-DHB_PROBES"]
    # (built beside the target and moved into place, so a reader never sees a half-written library)
    tmp = TARGET + ".tmp.%d" % os.getpid()
    cmd = [nvcc()] + NVCC_FLAGS + list(extra_flags) + ["-o", tmp] + SOURCES
    if verbose:
        print(" ".join(cmd))
    try:
        subprocess.check_call(cmd)
        os.replace(tmp, TARGET)
    finally:
        if os.path.exists(tmp):
            os.remove(tmp)
    return TARGET


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose=True,
          extra_flags=["-Xptxas", "-v"] if "--verbose" in sys.argv else [])
