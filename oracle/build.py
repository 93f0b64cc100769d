"""Builds the C oracle (oracle.c) into oracle/_build/liboracle.so with gcc + OpenMP.

The oracle is test infrastructure; building it is part of the repository's build check
but nothing in the shipped package loads the result.
"""
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_build", "liboracle.so")


def build(force: bool = False) -> str:
    src = os.path.join(HERE, "oracle.c")
    if not force and os.path.exists(OUT) and os.path.getmtime(OUT) >= os.path.getmtime(src):
        return OUT
    os.makedirs(os.path.dirname(OUT), exist_ok=True)
    cmd = ["gcc", "-O2", "-fopenmp", "-shared", "-fPIC", "-ffp-contract=off", "-mf16c", "-mfma",
           "-o", OUT, src, "-lm"]
    subprocess.run(cmd, check=True)
    return OUT


if __name__ == "__main__":
    print(build(force=True))
