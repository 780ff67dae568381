"""Compiles the reference's own CUDA kernels for cross-checks (test infrastructure).

The three kernel files of ug-llama that compile on their own (softmax.cu,
rope.cu, cat.cu) are built FROM WHERE THEY LIE in the reference tree, together
with the launchers of ``ref_cuda_launch.cu``, into ``oracle/_ref/libugref_cuda.so``.
No reference source is copied into this repository; ``oracle/_ref/`` is not
tracked.  The rest of the reference is Rust and cannot be built here (no
cargo / rustc in the image).  Without the reference tree this script does
nothing and the tests that need the library skip.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
# the reference checkout: $UG_REFERENCE_DIR, else a directory named "reference" beside this repository
REF = os.environ.get("UG_REFERENCE_DIR") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
OUT_DIR = os.path.join(HERE, "_ref")
OUT = os.path.join(OUT_DIR, "libugref_cuda.so")


def build(verbose=False):
    src_dir = os.path.join(REF, "ug-llama", "src")
    if not os.path.exists(os.path.join(src_dir, "softmax.cu")):
        return None
    os.makedirs(OUT_DIR, exist_ok=True)
    launcher = os.path.join(HERE, "ref_cuda_launch.cu")
    if os.path.exists(OUT) and os.path.getmtime(OUT) > os.path.getmtime(launcher):
        return OUT
    cmd = [os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc"), "-gencode", "arch=compute_100a,code=sm_100a", "-O3",
           "--use_fast_math", "-shared", "-Xcompiler", "-fPIC", "-cudart", "static", "-I", src_dir, launcher, "-o", OUT]
    if verbose:
        print(" ".join(cmd))
    subprocess.check_call(cmd)
    return OUT


if __name__ == "__main__":
    print(build(verbose=True))
