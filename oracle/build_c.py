"""Compile the plain-C restatement (oracle/spion_oracle.c) into oracle/_build/ (test infrastructure only).

    python oracle/build_c.py [--force]

Generic x86-64 code (no -march): the library is built where the compiler is and may be loaded on another host.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "spion_oracle.c")
OUT_DIR = os.path.join(HERE, "_build")
OUT = os.path.join(OUT_DIR, "libspion_oracle.so")
CC = os.environ.get("CC", "gcc")


def build(force=False):
    if not force and os.path.exists(OUT) and os.path.getmtime(OUT) >= os.path.getmtime(SRC):
        return OUT
    os.makedirs(OUT_DIR, exist_ok=True)
    cmd = [CC, "-O3", "-std=c99", "-fopenmp", "-fPIC", "-shared", "-Wall", "-Wextra", SRC, "-o", OUT, "-lm"]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout)
        raise RuntimeError("could not compile " + SRC)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
