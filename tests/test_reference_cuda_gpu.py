"""This backend's kernels against the REFERENCE'S OWN CUDA kernels
(ug-llama/src/softmax.cu, rope.cu, cat.cu compiled as they are into
oracle/_ref/ by oracle/build_ref.py) on the same device and inputs.  The
reference builds them with fast-math, so only the copy kernel is bit-exact;
rope agrees within an fma rounding, softmax within the error of __expf."""
import numpy as np
import pytest

import oracle
from conftest import rel_err
from ug_b200 import DType, synth
from ug_b200._lib import lib as ugb

pytestmark = pytest.mark.gpu
ref = oracle.reference_cuda()
needs_ref = pytest.mark.skipif(ref is None, reason="oracle/_ref/libugref_cuda.so was not built (no reference tree at build time)")


def rope_tables(max_pos, d, theta=10000.0):
    inv = np.array([1.0 / theta ** (i / d) for i in range(0, d, 2)], dtype=np.float32)
    ang = np.arange(max_pos, dtype=np.float32)[:, None] * inv[None, :]
    return np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)


@needs_ref
@pytest.mark.parametrize("rows,cols", [(2, 4), (64, 128), (33, 1000), (16, 4096), (5, 32000)])
def test_softmax_vs_reference_kernel(dev, rows, cols):
    x = synth.normal(40 + cols, (rows, cols), 2.0)
    src = dev.slice_from_values(x)
    mine, theirs = dev.allocate_uninit(DType.F32, x.size), dev.allocate_uninit(DType.F32, x.size)
    dev.custom_softmax(src, mine, rows, cols)
    assert ref.ugref_softmax_f32(src.device_ptr, theirs.device_ptr, rows, cols, ugb.ugb_device_stream(dev._h)) == 0
    dev.synchronize()
    a, b = mine.to_vec(), theirs.to_vec()
    assert rel_err(a, b) < 2e-5
    assert rel_err(a, oracle.custom_softmax(x).ravel()) < 1e-5       # and mine is the closer one to the CPU path


@needs_ref
@pytest.mark.parametrize("b,h,t,d,pos", [(1, 32, 1, 64, 0), (2, 4, 7, 64, 2040), (3, 2, 5, 16, 9)])
def test_rope_vs_reference_kernel(dev, b, h, t, d, pos):
    x = synth.normal(50 + t, (b, h, t, d))
    cos, sin = rope_tables(pos + t + 1, d)
    xs, cs, ss = (dev.slice_from_values(v) for v in (x, cos, sin))
    ps = dev.slice_from_values(np.array([pos], np.int32))
    mine, theirs = dev.allocate_uninit(DType.F32, x.size), dev.allocate_uninit(DType.F32, x.size)
    dev.rope(xs, cs, ss, ps, mine, b, h, t, d)
    assert ref.ugref_rope_f32(xs.device_ptr, cs.device_ptr, ss.device_ptr, ps.device_ptr, theirs.device_ptr, b, h, t, d,
                              ugb.ugb_device_stream(dev._h)) == 0
    dev.synchronize()
    assert np.max(np.abs(mine.to_vec() - theirs.to_vec())) < 1e-6 * max(1.0, float(np.abs(x).max()))


@needs_ref
@pytest.mark.parametrize("d1,d2_l,d2_r", [(4, 0, 64), (4, 2047 * 64, 64), (32, 16 * 64, 5 * 64), (3, 5, 2)])
def test_cat_vs_reference_kernel_bit_exact(dev, d1, d2_l, d2_r):
    lhs, rhs = synth.normal(60, (d1, d2_l)), synth.normal(61, (d1, d2_r))
    ls, rs = dev.slice_from_values(lhs), dev.slice_from_values(rhs)
    n = d1 * (d2_l + d2_r)
    mine, theirs = dev.allocate_uninit(DType.F32, n), dev.allocate_uninit(DType.F32, n)
    dev.cat(ls, rs, mine, d1, d2_l, d2_r)
    assert ref.ugref_cat_f32(ls.device_ptr, rs.device_ptr, theirs.device_ptr, d1, d2_l, d2_r, ugb.ugb_device_stream(dev._h)) == 0
    dev.synchronize()
    assert np.array_equal(mine.to_vec(), theirs.to_vec())
