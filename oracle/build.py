"""Compile the CPU checker into oracle/_build/libftm_oracle.so (test infrastructure).

Also, when the reference checkout is mounted and has sources that compile on
their own, this is where a recipe for oracle/_ref would live.  The reference is
a Rust crate (plus Triton kernels); no Rust toolchain exists in this image, so
nothing is built into oracle/_ref and the restatement is pinned by the
reference's known-answer tests and by fixtures from its Python torch oracle.
"""
from __future__ import annotations

import os
import shutil
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_build", "libftm_oracle.so")
SOURCES = [os.path.join(HERE, "ftm_oracle.c"), os.path.join(HERE, "ftm_oracle.h"),
           os.path.join(HERE, "..", "include", "ftm_exact_math.h")]
CFLAGS = ["-O2", "-march=x86-64-v3", "-ffp-contract=off", "-fno-fast-math", "-fopenmp", "-fPIC",
          "-Wall", "-Wextra", "-std=c11"]


def stale() -> bool:
    if not os.path.exists(OUT):
        return True
    t = os.path.getmtime(OUT)
    return any(os.path.getmtime(s) > t for s in SOURCES)


def build(force: bool = False) -> str:
    if not force and not stale():
        return OUT
    gcc = "/usr/bin/gcc" if os.path.exists("/usr/bin/gcc") else shutil.which("gcc")
    if gcc is None:
        raise RuntimeError("no gcc to build the CPU checker")
    os.makedirs(os.path.dirname(OUT), exist_ok=True)
    cmd = [gcc, *CFLAGS, "-shared", "-o", OUT, SOURCES[0], "-lm"]
    subprocess.run(cmd, check=True, cwd=HERE)
    return OUT


if __name__ == "__main__":
    print(build(force=True))
