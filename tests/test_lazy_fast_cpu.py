"""The generator of vectorised row / map kernels (host layer, ug_fast.cpp) without a GPU: the CUDA C it emits
for the graph forms of ug-llama/src/model.rs:65-109 compiles for sm_100a, uses 128-bit accesses, and shapes
it cannot express are declined (they take the SSA path)."""
import os
import subprocess
import tempfile

import numpy as np
import pytest

import oracle
from ug_b200 import llama_graph as G
from ug_b200 import synth
from ug_b200.lazy import LB, BinaryOp as B, Schedule

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")


@pytest.fixture(scope="module")
def hd():
    return oracle.cpu_host_device()


def sources(y):
    s = Schedule.create_one(y)
    return [s.fast_source(i) for i, kind in enumerate(s.items()) if kind == "Kernel"]


def compiles(src):
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "k.cu")
        open(path, "w").write(src)
        r = subprocess.run([NVCC, "-gencode", "arch=compute_100a,code=sm_100a", "--use_fast_math", "-c", path, "-o",
                            os.path.join(d, "k.o")], capture_output=True, text=True)
        assert r.returncode == 0, r.stderr


def test_row_and_map_kernels_are_generated_and_compile(hd):
    x, a = synth.normal(1, (16, 4096)), synth.uniform(2, (4096,), 0.5, 1.5)
    lx, la = LB.copy(x, x.shape, hd), LB.copy(a, a.shape, hd)
    (rms,) = sources(G.rms_norm(lx, la, 1e-5))
    assert rms.startswith("// row_vec4") and "float4" in rms and "__shfl_xor_sync" in rms
    compiles(rms)
    soft = sources(G.softmax(lx))            # two kernels under the CPU device's (= the reference's) cut rule
    assert len(soft) == 2 and all(s.startswith("// row_vec4") for s in soft)
    compiles(soft[0])
    (m,) = sources(G.silu(lx).binary(B.Mul, lx))
    assert m.startswith("// map_vec4")
    compiles(m)
    k = LB.copy(synth.normal(3, (1, 4, 9, 64)), (1, 4, 9, 64), hd)
    (rep,) = sources(G.repeat(k, 1, 8))
    assert rep.startswith("// warp_row_vec4") and "/ 8L" in rep        # the head index divided by n_rep
    compiles(rep)
    wide = sources(G.softmax(LB.copy(synth.normal(4, (2, 32000)), (2, 32000), hd)))[1]
    assert "block 1024" in wide.split("\n")[0]
    compiles(wide)


def test_rows_without_a_128_bit_form_and_shapes_that_are_declined(hd):
    y = LB.copy(synth.normal(5, (5, 777)), (5, 777), hd)
    soft = sources(G.softmax(y))                                        # 777 % 4 != 0: one element per access
    assert len(soft) == 2 and all(s.startswith("// row_scalar") and "float4" not in s.split("extern")[1] for s in soft)
    compiles(soft[0])
    # the head merge of model.rs:243 ([.., heads, 64] -> [.., heads * 64]): the column splits into (col / 64, col % 64)
    a = LB.copy(synth.normal(7, (1, 4, 8, 64)), (1, 4, 8, 64), hd)
    (merge,) = sources(a.transpose(2, 1).merge_dims(-2))
    assert merge.startswith("// warp_row_vec4") and "/ 64L" in merge and "% 64L" in merge
    compiles(merge)
    x = LB.copy(synth.normal(6, (8, 64)), (8, 64), hd)
    assert sources(x.reduce(0, 0)) == [""]                              # a reduction over the leading dim: SSA path
