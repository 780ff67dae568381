"""In-tree build of libugb200.so (sm_100a only).

``python -m ug_b200.build`` or ``ug_b200.build.build()`` compiles every
``csrc/*.cu`` with nvcc for ``compute_100a/sm_100a`` and links them into
``ug_b200/libugb200.so`` next to this file, so the binary travels with the
source tree.  nvcc cross-compiles without a GPU.
"""
import glob
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libugb200.so")

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
CFLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC,-fvisibility=hidden",
          "--expt-relaxed-constexpr", "-Xptxas", "-v"]


def _stale(out, deps):
    if not os.path.exists(out):
        return True
    t = os.path.getmtime(out)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False):
    """Compile and link; returns the path of the shared library."""
    os.makedirs(OBJ, exist_ok=True)
    srcs = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    hdrs = glob.glob(os.path.join(CSRC, "*.h")) + glob.glob(os.path.join(CSRC, "*.cuh")) + \
        glob.glob(os.path.join(HERE, "..", "include", "*.h"))
    objs, jobs = [], []
    for s in srcs:
        o = os.path.join(OBJ, os.path.basename(s)[:-3] + ".o")
        objs.append(o)
        if force or _stale(o, [s] + hdrs):
            jobs.append((s, o))

    def compile_one(job):
        s, o = job
        cmd = [NVCC] + ARCH + CFLAGS + ["-c", s, "-o", o]
        r = subprocess.run(cmd, capture_output=True, text=True)
        log = o[:-2] + ".ptxas.txt"
        with open(log, "w") as f:
            f.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {s}:\n{r.stdout}\n{r.stderr}")
        if verbose:
            print(f"compiled {os.path.basename(s)}")

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        list(ex.map(compile_one, jobs))
    if force or jobs or _stale(LIB, objs):
        cmd = [NVCC] + ARCH + ["-shared", "-o", LIB] + objs + ["-cudart", "static", "-ldl"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
        if verbose:
            print(f"linked {LIB}")
    build_host(force=force or bool(jobs), verbose=verbose)
    return LIB


HOST_DIR = os.path.join(CSRC, "host")
HOST_LIB = os.path.join(HERE, "libughost.so")


def build_host(force=False, verbose=False):
    """g++ build of the host layer (lazy graph, scheduler, lowering) against libugb200.so."""
    srcs = sorted(glob.glob(os.path.join(HOST_DIR, "*.cpp")))
    deps = srcs + glob.glob(os.path.join(HOST_DIR, "*.hpp")) + glob.glob(os.path.join(HERE, "..", "include", "*.h")) + [LIB]
    if not (force or _stale(HOST_LIB, deps)):
        return HOST_LIB
    cmd = ["g++", "-std=c++17", "-O2", "-fPIC", "-shared", "-fvisibility=hidden", "-Wall", "-Wextra"] + srcs + \
          ["-o", HOST_LIB, "-L" + HERE, "-lugb200", "-Wl,-rpath,$ORIGIN"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"host layer build failed:\n{r.stdout}\n{r.stderr}")
    if verbose:
        print(f"linked {HOST_LIB}")
    return HOST_LIB


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose=True)
