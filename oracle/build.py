"""Build recipe of the CPU oracle (test infrastructure, never shipped).

`python oracle/build.py` compiles oracle/fil_oracle.c into oracle/_build/libfil_oracle.so with
gcc and OpenMP.  The reference's own CPU implementation of this path is not compilable here: its
sources (nvForest, Treelite) are not vendored in the reference tree, so no oracle/_ref is built.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_build")
LIB = os.path.join(OUT_DIR, "libfil_oracle.so")
SOURCES = [os.path.join(HERE, "fil_oracle.c"), os.path.join(HERE, "fil_oracle_impl.h"),
           os.path.join(HERE, "..", "include", "b2fil.h")]


def build(force: bool = False) -> str:
    os.makedirs(OUT_DIR, exist_ok=True)
    if not force and os.path.exists(LIB):
        if all(not os.path.exists(s) or os.path.getmtime(s) <= os.path.getmtime(LIB)
               for s in SOURCES):
            return LIB
    if not os.path.exists(SOURCES[0]):
        raise RuntimeError("oracle sources missing")
    cmd = ["gcc", "-O3", "-march=x86-64-v2", "-fopenmp", "-fno-fast-math", "-shared", "-fPIC",
           "-o", LIB, SOURCES[0], "-lm"]
    subprocess.check_call(cmd)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
