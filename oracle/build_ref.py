"""Compile the reference's own CUDA files into oracle/_ref/ (test infrastructure only).

    python oracle/build_ref.py [/path/to/SPION]

The four files of the reference (models/attn.cu, attn_mask.cu, block_attn.cu,
block_attn_mask.cu) are compiled where they lie, with the reference's own command lines
(compile.sh:2-5) plus an explicit sm_100a target and an rpath to the CUDA libraries; nothing is
copied.  The resulting shared objects are used by tests/test_gpu_vs_reference_cuda.py to compare
this library with the reference's cuSPARSE / cuBLAS path on a GPU.  oracle/_ref/ is git-ignored.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
# where the reference checkout lies unless a path is given: $SPION_REFERENCE_ROOT, else ~/reference
DEFAULT_ROOT = os.environ.get("SPION_REFERENCE_ROOT", os.path.join(os.path.expanduser("~"), "reference"))
FILES = {"attn": "-lcublas", "attn_mask": "-lcublas", "block_attn": "-lcusparse", "block_attn_mask": "-lcusparse"}


def build(ref_root=DEFAULT_ROOT, force=False):
    if not os.path.isdir(os.path.join(ref_root, "models")):
        return []
    os.makedirs(OUT, exist_ok=True)
    built = []
    for name, libflag in FILES.items():
        src = os.path.join(ref_root, "models", name + ".cu")
        out = os.path.join(OUT, name + ".so")
        if force or not os.path.exists(out) or os.path.getmtime(out) < os.path.getmtime(src):
            cmd = [NVCC, "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC", "-shared", libflag,
                   "-Xlinker", "-rpath=/usr/local/cuda/lib64", "-o", out, src]
            r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
            if r.returncode != 0:
                sys.stderr.write(r.stdout)
                raise RuntimeError("could not compile " + src)
        built.append(out)
    return built


if __name__ == "__main__":
    roots = [a for a in sys.argv[1:] if not a.startswith("-")]
    print("\n".join(build(roots[0] if roots else DEFAULT_ROOT, force="--force" in sys.argv)))
