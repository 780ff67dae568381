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
    elif dtype == DType.F16:
        sa, sb = dev.slice_from_values(a.astype(np.float16)), dev.slice_from_values(b.astype(np.float16))
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
    return out.astype(np.float32).reshape(bs, m, n)


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


# ---- tcgen05 tensor-core path (bf16, row-major lhs, m*n >= 128*64) ---------
TC_SHAPES = [
    # bs, m, n, k, transpose_rhs
    (1, 128, 256, 64, True), (1, 128, 256, 64, False),        # one tile, one k block
    (1, 128, 256, 512, True), (1, 128, 256, 512, False),      # pipeline wraps (8 k blocks, 4 stages)
    (1, 256, 512, 256, True), (1, 256, 512, 256, False),      # 2x2 tiles
    (1, 200, 264, 200, True), (1, 200, 264, 200, False),      # ragged m, n, k tails
    (1, 64, 2048, 2048, True),                                # decode-shaped projection
    (3, 160, 320, 136, True), (3, 160, 320, 136, False),      # per-batch rhs
    (1, 2048, 1024, 1024, True), (1, 1024, 2048, 1024, False),  # many tiles per CTA (persistent loop)
]


@pytest.mark.parametrize("bs,m,n,k,t", TC_SHAPES)
def test_bf16_tensor_core_matmul(dev, bs, m, n, k, t):
    a = oracle.round_bf16(synth.normal(920 + m, (bs, m, k), 0.5))
    b = oracle.round_bf16(synth.normal(921 + n, (bs, n, k) if t else (bs, k, n), 0.5))
    got = gpu_matmul(dev, a, b, t, DType.BF16)
    ref = oracle.matmul(a, b, transpose_rhs=t)
    err = np.abs(got - ref) / np.maximum(np.abs(ref), 0.05 * np.abs(ref).max())
    assert err.max() < 2e-2
    # and the mean error must look like bf16 rounding of an exact f32 sum, not like a dropped k block
    assert np.abs(got - oracle.round_bf16(ref)).mean() < 2e-3 * np.abs(ref).mean()


@pytest.mark.parametrize("bs,m,n,k,t", TC_SHAPES)
def test_f16_tensor_core_matmul(dev, bs, m, n, k, t):
    """IEEE f16 operands on the same tcgen05 kernel (the instruction's format field is the only difference;
    the reference sends f16 to cublasGemmStridedBatchedEx like bf16, ug-cuda/src/gemm.rs:130-232)."""
    a = synth.normal(950 + m, (bs, m, k), 0.5).astype(np.float16).astype(np.float32)
    b = synth.normal(951 + n, (bs, n, k) if t else (bs, k, n), 0.5).astype(np.float16).astype(np.float32)
    got = gpu_matmul(dev, a, b, t, DType.F16)
    ref = oracle.matmul(a, b, transpose_rhs=t)
    err = np.abs(got - ref) / np.maximum(np.abs(ref), 0.05 * np.abs(ref).max())
    assert err.max() < 4e-3                       # f16 keeps 11 significant bits: 8x tighter than bf16's 2e-2
    assert np.abs(got - ref.astype(np.float16).astype(np.float32)).mean() < 3e-4 * np.abs(ref).mean()


# ---- f32 on the FP32 pipe: the skinny (decode) kernel and the 128 x 128 register-blocked kernel ----------------
@pytest.mark.parametrize("bs,m,n,k,t", [
    (1, 1, 2048, 2048, True), (1, 3, 5632, 2048, True), (2, 16, 264, 512, True), (1, 8, 32000, 256, True),   # skinny
    (1, 130, 200, 72, True), (1, 130, 200, 72, False), (2, 256, 384, 128, True), (1, 512, 2048, 2048, True),  # tiles
    (1, 127, 129, 67, False), (1, 17, 1031, 259, True),                                                       # no 128-bit form
    (32, 1, 64, 1029, False), (3, 5, 132, 37, False), (2, 8, 4, 1, False), (1, 2, 260, 2049, False)])        # skinny, n contiguous
def test_f32_matmul_kernels(dev, bs, m, n, k, t):
    a = synth.normal(960 + m, (bs, m, k))
    b = synth.normal(961 + n, (bs, n, k) if t else (bs, k, n))
    got = gpu_matmul(dev, a, b, t, DType.F32)
    ref = oracle.matmul(a, b, transpose_rhs=t) if m * n * k < 5e8 else np.matmul(a, np.swapaxes(b, -1, -2) if t else b)
    assert np.max(np.abs(got - ref)) / np.sqrt(k) < 1e-5     # fp32 products and sums, another order than the oracle


def test_f32_transposed_lhs(dev):
    """lhs stored [k, m] (its transpose is what the product reads): gemm.rs:18-43 accepts it."""
    bs, m, n, k = 1, 96, 136, 64
    a = synth.normal(970, (bs, m, k))
    b = synth.normal(971, (bs, k, n))
    at = np.ascontiguousarray(a.transpose(0, 2, 1))            # [k, m] in memory
    sa, sb = dev.slice_from_values(at), dev.slice_from_values(b)
    dst = dev.allocate_uninit(DType.F32, bs * m * n)
    dev.matmul(dst, sa, sb, (bs, m, n, k), transposed(contiguous(at.shape)), contiguous(b.shape))
    dev.synchronize()
    assert np.max(np.abs(dst.to_vec().reshape(bs, m, n) - oracle.matmul(a, b))) / np.sqrt(k) < 1e-5


def test_bf16_shared_weight_batch_is_flattened(dev):
    # [b, m, k] x shared [n, k] weight (batch stride 0), the Linear::fwd shape for b > 1
    bs, m, n, k = 4, 96, 256, 128
    a = oracle.round_bf16(synth.normal(930, (bs, m, k), 0.5))
    w = oracle.round_bf16(synth.normal(931, (n, k), 0.5))
    sa = dev.slice_from_values(synth.to_bf16_bits(a), bf16=True)
    sw = dev.slice_from_values(synth.to_bf16_bits(w), bf16=True)
    dst = dev.allocate_uninit(DType.BF16, bs * m * n)
    dev.matmul(dst, sa, sw, (bs, m, n, k), contiguous((bs, m, k)), ([bs, k, n], [0, 1, k], 0))
    dev.synchronize()
    got = synth.bf16_bits_to_f32(dst.to_vec()).reshape(bs, m, n)
    ref = oracle.matmul(a, w, transpose_rhs=True)
    assert np.max(np.abs(got - ref)) / np.abs(ref).max() < 2e-2


def test_bf16_config3_full_size_sampled_rows_and_linearity(dev):
    """Config 3: A [16,512,4096] x B [4096,4096] ([k,n] layout), bf16, fp32 accumulate."""
    bs, m, n, k = 16, 512, 4096, 4096
    a = oracle.round_bf16(synth.normal(4, (bs, m, k), 0.02))
    b = oracle.round_bf16(synth.normal(5, (k, n), 0.02))
    sa = dev.slice_from_values(synth.to_bf16_bits(a), bf16=True)
    sb = dev.slice_from_values(synth.to_bf16_bits(b), bf16=True)
    dst = dev.allocate_uninit(DType.BF16, bs * m * n)
    dev.matmul(dst, sa, sb, (bs, m, n, k), contiguous((bs, m, k)), ([bs, k, n], [0, n, 1], 0))
    dev.synchronize()
    got = synth.bf16_bits_to_f32(dst.to_vec()).reshape(bs * m, n)
    rows = np.r_[0:8, 127:130, 4095:4098, 8184:8192]           # tile edges, batch edges, last rows
    ref = oracle.matmul(a.reshape(bs * m, k)[rows], b)
    err = np.abs(got[rows] - ref) / np.maximum(np.abs(ref), 0.05 * np.abs(ref).max())
    assert err.max() < 2e-2
    # size-independent property over the whole output: (1^T A) B == 1^T (A B) column sums
    col_ref = (a.reshape(-1, k).astype(np.float64).sum(0)) @ b.astype(np.float64)
    col_got = got.astype(np.float64).sum(0)
    assert np.max(np.abs(col_got - col_ref)) < 5e-3 * np.abs(col_ref).max() + 0.5


# ---- CTA pairs (tcgen05 cta_group::2): 256 x 256 tiles on two SMs ---------------------------------------------
PAIR_SHAPES = [
    (1, 256, 256, 64, True), (1, 256, 256, 64, False),        # one tile, one k block
    (1, 256, 256, 1024, True), (1, 256, 256, 1024, False),    # the 6-stage ring wraps (16 k blocks)
    (1, 200, 264, 200, True), (1, 200, 264, 200, False),      # ragged m (second CTA partly empty), n, k tails
    (1, 129, 128, 72, True),                                  # one row in the second CTA, half an n tile
    (3, 160, 320, 136, True), (3, 160, 320, 136, False),      # per-batch rhs
    (1, 4096, 2048, 512, True), (1, 2048, 4096, 256, False),  # more tiles than clusters (persistent loop), both tile orders
]


@pytest.mark.parametrize("bs,m,n,k,t", PAIR_SHAPES)
def test_bf16_matmul_on_cta_pairs_matches_single_ctas(dev, bs, m, n, k, t):
    """The pair kernel accumulates every output element over k in the same order as the single-CTA kernel: the
    results agree bit for bit, and with the oracle within the bf16 tolerance."""
    a = oracle.round_bf16(synth.normal(940 + m, (bs, m, k), 0.5))
    b = oracle.round_bf16(synth.normal(941 + n, (bs, n, k) if t else (bs, k, n), 0.5))
    dev.set_option("gemm_cta_pairs", 0)
    single = gpu_matmul(dev, a, b, t, DType.BF16)
    try:
        dev.set_option("gemm_cta_pairs", 1)
        pair = gpu_matmul(dev, a, b, t, DType.BF16)
    finally:
        dev.set_option("gemm_cta_pairs", 1)      # the default
    ref = oracle.matmul(a, b, transpose_rhs=t)
    err = np.abs(pair - ref) / np.maximum(np.abs(ref), 0.05 * np.abs(ref).max())
    assert err.max() < 2e-2
    assert np.array_equal(pair, single)


def test_device_option_errors(dev):
    with pytest.raises(UgError):
        dev.set_option("gemm_cta_pairs", 2)
    with pytest.raises(UgError):
        dev.set_option("no_such_option", 1)
