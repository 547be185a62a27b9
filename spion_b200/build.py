"""Build the CUDA library in-tree for sm_100a (nvcc cross-compiles without a GPU).

    python -m spion_b200.build [--force]

Outputs (git-ignored, but shipped with the working tree):
    spion_b200/lib/libspion_b200.so        all kernels + the C ABI of include/spion_b200.h
    spion_b200/lib/{attn,attn_mask,block_attn,block_attn_mask}.so
                                           shims with the reference's own symbol names
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "lib")
OBJ = os.path.join(HERE, "build")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
CUFLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--fmad=true", "-Xptxas", "-v"]
SHIMS = {"attn": 0, "attn_mask": 1, "block_attn": 2, "block_attn_mask": 3}


def _newer(src_list, out):
    if not os.path.exists(out):
        return True
    t = os.path.getmtime(out)
    return any(os.path.getmtime(s) > t for s in src_list)


def _run(cmd, log=None):
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if log is not None:
        with open(log, "w") as f:
            f.write(" ".join(cmd) + "\n" + r.stdout)
    if r.returncode != 0:
        sys.stderr.write(r.stdout)
        raise RuntimeError("build step failed: " + " ".join(cmd))
    return r.stdout


def build_all(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(LIB, exist_ok=True)
    os.makedirs(OBJ, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    headers.append(os.path.join(os.path.dirname(HERE), "include", "spion_b200.h"))
    cus = sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))
    objs = []
    for f in cus:
        src = os.path.join(CSRC, f)
        obj = os.path.join(OBJ, f[:-3] + ".o")
        objs.append(obj)
        if force or _newer([src] + headers, obj):
            out = _run([NVCC] + ARCH + CUFLAGS + ["-c", src, "-o", obj], log=obj + ".log")
            if verbose:
                print(out)
    main = os.path.join(LIB, "libspion_b200.so")
    if force or _newer(objs, main):
        _run([NVCC] + ARCH + ["-shared", "-o", main] + objs + ["-lcudart_static", "-lpthread", "-ldl", "-lrt"])
    shim_src = os.path.join(CSRC, "shim.cpp")
    for name, kind in SHIMS.items():
        out = os.path.join(LIB, name + ".so")
        if force or _newer([shim_src, main] + headers, out):
            _run(["g++", "-O2", "-fPIC", "-shared", f"-DSPION_SHIM_KIND={kind}", shim_src, "-o", out,
                  "-L" + LIB, "-lspion_b200", "-Wl,-rpath,$ORIGIN"])
    return main


if __name__ == "__main__":
    print(build_all(force="--force" in sys.argv, verbose="-v" in sys.argv))
