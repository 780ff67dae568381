"""GPU parity of the fused row operators against the CPU oracle, through the
C ABI.  Tolerance for fp32 reductions: 1e-5 relative (the oracle's emitted-C
form is itself built with -ffast-math, so bit-exactness is not defined)."""
import numpy as np
import pytest

import oracle
from conftest import rel_err
from ug_b200 import DType, UgError, synth

pytestmark = pytest.mark.gpu
TOL = 1e-5

GOLD_IN = np.array([[0., 1., 2., 3.], [2., 1., 2., 1.]], dtype=np.float32)
GOLD_OUT = np.array([0.032058604, 0.08714432, 0.23688284, 0.6439143,
                     0.3655293, 0.13447072, 0.3655293, 0.13447072], dtype=np.float32)


def run_softmax(dev, x):
    n_cols = x.shape[-1]
    src = dev.slice_from_values(x)
    dst = dev.allocate_uninit(DType.F32, x.size)
    dev.custom_softmax(src, dst, x.size // n_cols if n_cols else 0, n_cols)
    dev.synchronize()
    return dst.to_vec().reshape(x.shape)


def test_softmax_reference_known_answer(dev):
    # ug-core/tests/basic_tests.rs:41-116
    assert rel_err(run_softmax(dev, GOLD_IN).ravel(), GOLD_OUT) < 3e-7


# (rows, cols): warp-per-row, CTA-per-row at each register width, general path
# (odd length, > 8192, longer than the shared-memory cache), single row/col.
SHAPES = [(2, 4), (8, 4), (64, 128), (33, 256), (40, 1024), (7, 1028), (16, 2048), (5, 4096),
          (3, 8192), (9, 1000), (11, 1023), (3, 8196), (4, 32000), (2, 50001), (1, 1), (17, 1),
          (1, 4096)]


@pytest.mark.parametrize("rows,cols", SHAPES)
def test_softmax_shapes(dev, rows, cols):
    x = synth.normal(100 + rows + cols, (rows, cols), 2.0)
    got = run_softmax(dev, x)
    assert rel_err(got, oracle.custom_softmax(x)) < TOL
    if rows * cols * cols <= 2 ** 28:
        assert rel_err(got, oracle.gen_softmax(x)) < TOL
    assert np.allclose(got.sum(-1), 1.0, atol=1e-5)


def test_softmax_config1_full(dev):
    x = synth.softmax_c1()
    got = run_softmax(dev, x)
    assert rel_err(got, oracle.custom_softmax(x)) < TOL
    sub = oracle.gen_softmax(x, rows=(0, 32))[:32]   # the O(cols^2) lazy-graph form on a row subset
    assert rel_err(got[:32], sub) < TOL


def test_softmax_in_place_and_extremes(dev):
    x = synth.normal(7, (6, 512), 30.0)
    x[0, :] = -1e30
    x[1, 3] = 1e30
    x[2, :] = -np.inf
    x[2, 5] = 0.0
    s = dev.slice_from_values(x)
    dev.custom_softmax(s, s, 6, 512)
    dev.synchronize()
    got = s.to_vec().reshape(x.shape)
    ref = oracle.custom_softmax(x)
    assert np.all(np.isfinite(got))
    assert rel_err(got, ref, 1e-37) < TOL


def test_softmax_unaligned_base_pointer(dev):
    # a slice that starts 4 bytes into an allocation takes the scalar path
    import ctypes as C
    from ug_b200._lib import lib
    x = synth.normal(9, (5, 64), 2.0)
    big = dev.allocate_uninit(DType.F32, x.size + 1)
    out = dev.allocate_uninit(DType.F32, x.size + 1)
    h_in, h_out = C.c_void_p(), C.c_void_p()
    assert lib.ugb_wrap(dev._h, big.device_ptr + 4, int(DType.F32), x.size, C.byref(h_in)) == 0
    assert lib.ugb_wrap(dev._h, out.device_ptr + 4, int(DType.F32), x.size, C.byref(h_out)) == 0
    assert lib.ugb_h2d(h_in, x.ctypes.data, x.size, int(DType.F32)) == 0
    assert lib.ugb_softmax(dev._h, h_in, h_out, 5, 64) == 0
    got = np.empty_like(x)
    assert lib.ugb_d2h(h_out, got.ctypes.data, x.size, int(DType.F32)) == 0
    lib.ugb_free(h_in)
    lib.ugb_free(h_out)
    assert rel_err(got, oracle.custom_softmax(x)) < TOL


def test_zero_sized_rows_are_noops(dev):
    empty = dev.allocate_uninit(DType.F32, 0)
    assert empty.is_empty() and empty.device_ptr == 0
    n0 = dev.launch_count
    dev.custom_softmax(empty, empty, 0, 128)
    dev.custom_softmax(empty, empty, 5, 0)
    dev.synchronize()
    assert dev.launch_count == n0


RMS_SHAPES = [(4, 8), (64, 64), (19, 576), (8, 2048), (6, 4096), (2, 8192), (5, 2050), (3, 777),
              (2, 11008), (1, 5), (3, 45000)]


@pytest.mark.parametrize("rows,cols", RMS_SHAPES)
def test_rms_norm_shapes(dev, rows, cols):
    x = synth.normal(200 + cols, (rows, cols))
    w = synth.uniform(201 + cols, (cols,), 0.5, 1.5)
    xs, ws = dev.slice_from_values(x), dev.slice_from_values(w)
    dst = dev.allocate_uninit(DType.F32, x.size)
    dev.rms_norm(xs, ws, dst, rows, cols, 1e-5)
    dev.synchronize()
    got = dst.to_vec().reshape(x.shape)
    assert rel_err(got, oracle.gen_rms_norm(x, w, 1e-5), 1e-20) < TOL


@pytest.mark.parametrize("rows,cols", RMS_SHAPES)
def test_rms_norm_silu_gate_shapes(dev, rows, cols):
    x = synth.normal(300 + cols, (rows, cols))
    g = synth.normal(301 + cols, (rows, cols))
    w = synth.uniform(302 + cols, (cols,), 0.5, 1.5)
    xs, gs, ws = dev.slice_from_values(x), dev.slice_from_values(g), dev.slice_from_values(w)
    dst = dev.allocate_uninit(DType.F32, x.size)
    dev.rms_norm_silu_gate(xs, ws, gs, dst, rows, cols, 1e-5)
    dev.synchronize()
    got = dst.to_vec().reshape(x.shape)
    assert rel_err(got, oracle.gen_rms_norm_silu_gate(x, w, g, 1e-5), 1e-20) < TOL


def test_rms_silu_config2_full_size_properties(dev):
    """Config 2 at full size: oracle on a row subset + scale-invariance of rms_norm."""
    x, g, w, eps = synth.rms_silu_c2()
    rows, cols = x.shape
    xs, gs, ws = dev.slice_from_values(x), dev.slice_from_values(g), dev.slice_from_values(w)
    dst = dev.allocate_uninit(DType.F32, x.size)
    dev.rms_norm_silu_gate(xs, ws, gs, dst, rows, cols, eps)
    dev.synchronize()
    got = dst.to_vec().reshape(x.shape)
    for lo in (0, 4096, rows - 16):
        ref = oracle.gen_rms_norm_silu_gate(x, w, g, eps, rows=(lo, lo + 16))[lo:lo + 16]
        assert rel_err(got[lo:lo + 16], ref, 1e-20) < TOL
    # rms_norm(c * x) == rms_norm(x) up to the eps term: a size-independent check of every row
    xs2 = dev.slice_from_values(x * np.float32(4.0))
    dst2 = dev.allocate_uninit(DType.F32, x.size)
    dev.rms_norm_silu_gate(xs2, ws, gs, dst2, rows, cols, eps)
    dev.synchronize()
    got2 = dst2.to_vec().reshape(x.shape)
    assert np.allclose(got2, got, rtol=2e-5, atol=1e-7)


def test_dtype_and_length_errors(dev):
    a = dev.allocate_uninit(DType.F32, 16)
    i = dev.allocate_uninit(DType.I32, 16)
    with pytest.raises(UgError) as e:
        dev.custom_softmax(i, a, 4, 4)
    assert e.value.code == 2 and "dtype mismatch" in e.value.msg
    with pytest.raises(UgError) as e:
        dev.custom_softmax(a, a, 4, 8)
    assert e.value.code == 3
    with pytest.raises(UgError) as e:     # htod dtype check, ug-cuda/src/runtime.rs:376
        a.copy_host_to_device(np.zeros(16, np.int32))
    assert e.value.code == 2
    with pytest.raises(UgError) as e:     # length check
        a.copy_host_to_device(np.zeros(15, np.float32))
    assert e.value.code == 3
