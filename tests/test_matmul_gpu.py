"""GPU parity of ug::Device::matmul through the C ABI.

f32: against the oracle GEMM stand-in, <= 1e-5 relative to the row scale.
bf16: operands rounded to bf16 on the host, oracle in f32 on the rounded
values, result compared at <= 2e-2 relative (the stated bf16 tolerance)."""
import numpy as np
import pytest

import oracle
from ug_b200 import DType, UgError, synth

pytestmark = pytest.mark.gpu


def contiguous(shape):
    strides, acc = [], 1
    for d in reversed(shape):
        strides.append(acc)
        acc *= d
    return list(shape), list(reversed(strides)), 0


def transposed(layout):
    dims, strides, off = layout
    dims, strides = list(dims), list(strides)
    dims[-1], dims[-2] = dims[-2], dims[-1]
    strides[-1], strides[-2] = strides[-2], strides[-1]
    return dims, strides, off


def gpu_matmul(dev, a, b, transpose_rhs, dtype):
    """a [b,m,k]; b [b,k,n] or [b,n,k] if transpose_rhs.  Mirrors how the
    schedule calls Device::matmul (ug-core/src/schedule.rs:256-288)."""
    bs, m, k = a.shape
    n = b.shape[1] if transpose_rhs else b.shape[2]
    if dtype == DType.BF16:
        sa, sb = dev.slice_from_values(synth.to_bf16_bits(a), bf16=True), \
            dev.slice_from_values(synth.to_bf16_bits(b), bf16=True)
    else:
        sa, sb = dev.slice_from_values(a), dev.slice_from_values(b)
    dst = dev.allocate_uninit(dtype, bs * m * n)
    lhs_l = contiguous(a.shape)
    rhs_l = contiguous(b.shape)
    if transpose_rhs:
        rhs_l = transposed(rhs_l)
    dev.matmul(dst, sa, sb, (bs, m, n, k), lhs_l, rhs_l)
    dev.synchronize()
    out = dst.to_vec()
    if dtype == DType.BF16:
        out = synth.bf16_bits_to_f32(out)
    return out.reshape(bs, m, n)


def test_mm_reference_fixture(dev):
    # ug-core/src/common_tests.rs:15-22
    out = gpu_matmul(dev, np.full((1, 4, 2), 1.0, np.float32), np.full((1, 2, 3), 2.0, np.float32),
                     False, DType.F32)
    assert np.array_equal(out, np.full((1, 4, 3), 4.0, np.float32))


@pytest.mark.parametrize("bs,m,n,k,t", [(1, 4, 3, 2, False), (3, 17, 9, 33, False), (3, 17, 9, 33, True),
                                         (2, 64, 64, 64, True), (1, 130, 70, 257, False),
                                         (32, 1, 65, 64, True), (32, 1, 64, 65, False), (1, 2048, 1, 32, False)])
def test_f32_matmul(dev, bs, m, n, k, t):
    a = synth.normal(900, (bs, m, k))
    b = synth.normal(901, (bs, n, k) if t else (bs, k, n))
    got = gpu_matmul(dev, a, b, t, DType.F32)
    ref = oracle.matmul(a, b, transpose_rhs=t)
    scale = np.sqrt(k) * 1.0
    assert np.max(np.abs(got - ref)) / scale < 1e-5


def test_f32_rope_table_outer_product(dev):
    # ug-llama/src/model.rs:278-295: [max_pos, 1] . [1, d/2]; k == 1 products are exact
    theta = np.array([1.0 / 10000.0 ** (i / 64) for i in range(0, 64, 2)], np.float32)[None, None]
    idx = np.arange(4096, dtype=np.float32)[None, :, None]
    got = gpu_matmul(dev, idx, theta, False, DType.F32)
    assert np.array_equal(got[0], idx[0] * theta[0])


@pytest.mark.parametrize("bs,m,n,k,t", [(1, 5, 7, 9, True), (2, 33, 65, 100, False), (1, 64, 256, 2048, True)])
def test_bf16_matmul_small(dev, bs, m, n, k, t):
    a = oracle.round_bf16(synth.normal(910, (bs, m, k), 0.5))
    b = oracle.round_bf16(synth.normal(911, (bs, n, k) if t else (bs, k, n), 0.5))
    got = gpu_matmul(dev, a, b, t, DType.BF16)
    ref = oracle.matmul(a, b, transpose_rhs=t)
    scale = np.abs(ref).max()
    assert np.max(np.abs(got - ref)) / scale < 2e-2


def test_matmul_errors(dev):
    f = dev.allocate_uninit(DType.F32, 64)
    h = dev.allocate_uninit(DType.BF16, 64)
    i = dev.allocate_uninit(DType.I32, 64)
    lay = contiguous((1, 8, 8))
    with pytest.raises(UgError) as e:      # ug-cuda/src/gemm.rs:325-330
        dev.matmul(f, h, f, (1, 8, 8, 8), lay, lay)
    assert e.value.code == 2 and "incorrect dtypes for matmul" in e.value.msg
    with pytest.raises(UgError) as e:
        dev.matmul(i, i, i, (1, 8, 8, 8), lay, lay)
    assert e.value.code == 2
    bad = ([1, 8, 8], [64, 16, 2], 0)      # neither row-major nor its transpose: gemm.rs:32,42
    with pytest.raises(UgError) as e:
        dev.matmul(f, f, f, (1, 8, 8, 8), lay, bad)
    assert e.value.code == 3 and "non contiguous matmul" in e.value.msg
    with pytest.raises(UgError) as e:      # dst too small
        dev.matmul(f, f, f, (2, 8, 8, 8), contiguous((2, 8, 8)), contiguous((2, 8, 8)))
    assert e.value.code == 3
