"""Build recipe for the CPU oracle (test infrastructure, not product code).

Two translation units with different arithmetic rules:

* ``ug_cpu_gen.c``  -- the C that ug-core's CPU backend emits; compiled with
  the reference's exact command line (ug-core/src/cpu_runtime.rs:476-488):
  ``gcc -shared -lm -O3 -march=native -ffast-math -fomit-frame-pointer``.
* ``ug_cpu_ops.c`` / ``ug_llama_ref.c`` -- restatements of Rust code, which
  never reassociates nor contracts to FMA: ``-O3 -march=native
  -fno-fast-math -ffp-contract=off -fopenmp``.

``-march=native`` binds a binary to the CPU it was built on, so the output
name carries a hash of the host's CPU flags; a box with another CPU rebuilds
(gcc is part of the image) instead of loading a binary it cannot run.
"""
import hashlib
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_build")

GEN_FLAGS = ["-shared", "-lm", "-O3", "-march=native", "-ffast-math", "-fomit-frame-pointer"]
OPS_FLAGS = ["-shared", "-lm", "-O3", "-march=native", "-fno-fast-math", "-ffp-contract=off",
             "-fopenmp"]


def _cpu_tag():
    flags = ""
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("flags"):
                    flags = line
                    break
    except OSError:
        pass
    return hashlib.sha1(flags.encode()).hexdigest()[:10]


def _needs(out, srcs):
    if not os.path.exists(out):
        return True
    t = os.path.getmtime(out)
    return any(os.path.getmtime(s) > t for s in srcs)


def build(verbose=False):
    """Compile both oracle libraries if missing or stale; return their paths."""
    os.makedirs(OUT, exist_ok=True)
    tag = _cpu_tag()
    gen_so = os.path.join(OUT, f"libug_cpu_gen_{tag}.so")
    ops_so = os.path.join(OUT, f"libug_cpu_ops_{tag}.so")
    gen_src = [os.path.join(HERE, "ug_cpu_gen.c")]
    ops_src = [os.path.join(HERE, n) for n in ("ug_cpu_ops.c", "ug_llama_ref.c")
               if os.path.exists(os.path.join(HERE, n))]
    if _needs(gen_so, gen_src):
        cmd = ["gcc"] + gen_src + GEN_FLAGS + ["-fPIC", "-o", gen_so]
        if verbose:
            print(" ".join(cmd))
        subprocess.check_call(cmd)
    if _needs(ops_so, ops_src + [__file__]):
        cmd = ["gcc"] + ops_src + OPS_FLAGS + ["-fPIC", "-o", ops_so]
        if verbose:
            print(" ".join(cmd))
        subprocess.check_call(cmd)
    return gen_so, ops_so


def build_cpu_device(verbose=False):
    """ug-core's CPU backend behind the C++ ug::Device interface of the host layer (cpu_device.cpp),
    with the GEMM stand-in of ug_cpu_ops.c compiled in under its own arithmetic flags."""
    os.makedirs(OUT, exist_ok=True)
    tag = _cpu_tag()
    so = os.path.join(OUT, f"liboracle_cpudev_{tag}.so")
    cpp = os.path.join(HERE, "cpu_device.cpp")
    ops = os.path.join(HERE, "ug_cpu_ops.c")
    host_hdrs = [os.path.join(HERE, "..", "ug_b200", "csrc", "host", n)
                 for n in ("ug_core.hpp", "ug_lower.hpp", "ug_graph.hpp")]
    if _needs(so, [cpp, ops, __file__] + host_hdrs):
        obj = os.path.join(OUT, f"ug_cpu_ops_{tag}.o")
        c1 = ["gcc", "-c", ops, "-O3", "-march=native", "-fno-fast-math", "-ffp-contract=off", "-fopenmp", "-fPIC", "-o", obj]
        c2 = ["g++", "-std=c++17", "-O2", "-fPIC", "-shared", "-fvisibility=hidden", cpp, obj, "-o", so, "-fopenmp", "-ldl"]
        for c in (c1, c2):
            if verbose:
                print(" ".join(c))
            subprocess.check_call(c)
    return so


if __name__ == "__main__":
    print(build(verbose=True))
    print(build_cpu_device(verbose=True))
