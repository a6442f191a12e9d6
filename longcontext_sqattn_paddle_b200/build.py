"""Build libsqattn_b200.so in-tree with nvcc for sm_100a.

    python longcontext_sqattn_paddle_b200/build.py [--force] [--debug-exports]

(run as a script: it must work before the package itself can be imported)
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "csrc", "sqattn_b200.cu")
OUT = os.path.join(HERE, "libsqattn_b200.so")
DEPS = [os.path.join(HERE, "csrc", f) for f in os.listdir(os.path.join(HERE, "csrc"))]
DEPS.append(os.path.join(os.path.dirname(HERE), "include", "sqattn_b200.h"))


def nvcc_command(out=OUT, extra=()):
    return ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
            "-shared", "-Xcompiler", "-fPIC", *extra, "-o", out, SRC]


def up_to_date(out=OUT):
    if not os.path.exists(out):
        return False
    t = os.path.getmtime(out)
    return all(os.path.getmtime(d) <= t for d in DEPS)


def build(force=False, out=OUT, extra=(), verbose=False):
    if not force and up_to_date(out):
        return out
    cmd = nvcc_command(out, extra)
    if verbose:
        print(" ".join(cmd))
    subprocess.run(cmd, check=True)
    return out


DEBUG_OUT = os.path.join(HERE, "libsqattn_b200_debug.so")


def build_debug(force=False, verbose=False):
    """The same library with the debug exports (tile dumps, time stamps) that some tests and profiling probes read."""
    return build(force, DEBUG_OUT, ("-DSQATTN_DEBUG_EXPORTS",), verbose)


if __name__ == "__main__":
    if "--debug-exports" in sys.argv:
        build_debug(True, True)
    else:
        build("--force" in sys.argv, verbose=True)
