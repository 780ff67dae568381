"""GPU parity of ug-llama's custom operators and the gather / map kernels.
Copies, masks, gathers and the rope rotation are bit-exact against the CPU
oracle (ug-llama/src/cpu_ops.rs); silu*up is a fp32 map within 1e-5."""
import numpy as np
import pytest

import oracle
from conftest import rel_err
from ug_b200 import DType, UgError, synth

pytestmark = pytest.mark.gpu


def rope_tables(max_pos, d, theta=10000.0):
    inv = np.array([1.0 / theta ** (i / d) for i in range(0, d, 2)], dtype=np.float32)
    ang = np.arange(max_pos, dtype=np.float32)[:, None] * inv[None, :]
    return np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)


@pytest.mark.parametrize("interleaved", [False, True])
@pytest.mark.parametrize("b,h,t,d,pos", [(1, 32, 1, 64, 0), (1, 4, 1, 64, 2047), (8, 32, 16, 64, 5),
                                          (2, 3, 5, 16, 7), (1, 2, 3, 6, 1), (2, 2, 7, 2, 3),
                                          (4, 8, 128, 128, 100)])
def test_rope_bit_exact(dev, interleaved, b, h, t, d, pos):
    x = synth.normal(400 + d + t, (b, h, t, d))
    cos, sin = rope_tables(pos + t + 3, d)
    p = np.array([pos], np.int32)
    xs, cs, ss, ps = (dev.slice_from_values(v) for v in (x, cos, sin, p))
    dst = dev.allocate_uninit(DType.F32, x.size)
    (dev.rope_i if interleaved else dev.rope)(xs, cs, ss, ps, dst, b, h, t, d)
    dev.synchronize()
    ref = (oracle.rope_i if interleaved else oracle.rope)(x, cos, sin, p)
    assert np.array_equal(dst.to_vec().reshape(x.shape), ref)


def test_rope_rejects_odd_head_dim(dev):
    s = dev.allocate_uninit(DType.F32, 15)
    p = dev.allocate_uninit(DType.I32, 1)
    with pytest.raises(UgError) as e:
        dev.rope(s, s, s, p, s, 1, 1, 3, 5)
    assert e.value.code == 3


@pytest.mark.parametrize("l_shape,r_shape,axis", [
    ((1, 4, 0, 64), (1, 4, 1, 64), 2),        # first decode step: empty cache
    ((1, 4, 2047, 64), (1, 4, 1, 64), 2),     # KV append at T = 2047
    ((8, 4, 16, 64), (8, 4, 5, 64), 2),
    ((2, 2), (2, 2), 0), ((2, 2), (2, 2), 1), ((3, 5), (3, 2), 1), ((2, 3, 3), (2, 1, 3), 1)])
def test_cat_bit_exact(dev, l_shape, r_shape, axis):
    lhs = synth.normal(500 + axis, l_shape)
    rhs = synth.normal(501 + axis, r_shape)
    ref = oracle.cat(lhs, rhs, axis)
    d1 = int(np.prod(l_shape[:axis], dtype=np.int64))
    d2_l = int(np.prod(l_shape[axis:], dtype=np.int64))
    d2_r = int(np.prod(r_shape[axis:], dtype=np.int64))
    ls, rs = dev.slice_from_values(lhs), dev.slice_from_values(rhs)
    dst = dev.allocate_uninit(DType.F32, ref.size)
    dev.cat(ls, rs, dst, d1, d2_l, d2_r)
    dev.synchronize()
    assert np.array_equal(dst.to_vec().reshape(ref.shape), ref)


def test_cat_reference_fixture(dev):
    # ug-core/src/common_tests.rs:24-30, outer axis: [a0; a1; a2]
    a = [np.array(v, np.float32) for v in ([1., 2., 3., 4.], [1.1, 2.1, 3.1, 4.1], [1.2, 2.2, 3.2, 4.2])]
    s = [dev.slice_from_values(v) for v in a]
    t = dev.allocate_uninit(DType.F32, 8)
    dev.cat(s[0], s[1], t, 1, 4, 4)
    out = dev.allocate_uninit(DType.F32, 12)
    dev.cat(t, s[2], out, 1, 8, 4)
    dev.synchronize()
    assert np.array_equal(out.to_vec(), np.array(
        [1.0, 2.0, 3.0, 4.0, 1.1, 2.1, 3.1, 4.1, 1.2, 2.2, 3.2, 4.2], np.float32))


@pytest.mark.parametrize("b,h,s1,s2", [(1, 1, 3, 3), (2, 4, 16, 16), (1, 2, 7, 7), (1, 3, 5, 9),
                                        (2, 2, 64, 64), (1, 32, 512, 512), (1, 1, 6, 4)])
def test_causal_mask_bit_exact(dev, b, h, s1, s2):
    x = synth.normal(600 + s1, (b, h, s1, s2))
    src = dev.slice_from_values(x)
    dst = dev.allocate_uninit(DType.F32, x.size)
    dev.causal_mask(src, dst, b * h, s1, s2)
    dev.synchronize()
    assert np.array_equal(dst.to_vec().reshape(x.shape), oracle.causal_mask(x))


@pytest.mark.parametrize("vocab,h,ids_shape", [(10, 6, (2, 3)), (32000, 2048, (8, 64)), (50, 7, (1, 1)),
                                                (100, 64, (3, 0))])
def test_index_select_bit_exact(dev, vocab, h, ids_shape):
    emb = synth.normal(700, (vocab, h))
    ids = synth.tokens(701, ids_shape, vocab)
    es, is_ = dev.slice_from_values(emb), dev.slice_from_values(ids)
    dst = dev.allocate_uninit(DType.F32, ids.size * h)
    dev.index_select(es, is_, dst, ids.size, h, vocab)
    dev.synchronize()
    assert np.array_equal(dst.to_vec().reshape(ids.shape + (h,)), oracle.index_select(emb, ids))


def test_index_select_reports_bad_id_without_faulting(dev):
    emb = synth.normal(702, (10, 8))
    ids = np.array([1, 12, -3, 2], np.int32)
    es, is_ = dev.slice_from_values(emb), dev.slice_from_values(ids)
    dst = dev.slice_from_values(np.zeros(32, np.float32))
    dev.index_select(es, is_, dst, 4, 8, 10)
    with pytest.raises(UgError) as e:
        dev.synchronize()
    assert e.value.code == 1
    out = dst.to_vec().reshape(4, 8)
    assert np.array_equal(out[0], emb[1]) and np.array_equal(out[3], emb[2])
    assert not out[1].any() and not out[2].any()
    dev.synchronize()      # the status word was cleared: the device stays usable


@pytest.mark.parametrize("n", [1, 3, 4, 10, 5632, 64 * 5632, 1000003])
def test_add_and_silu_mul(dev, n):
    a, b = synth.normal(800, (n,)), synth.normal(801, (n,))
    sa, sb = dev.slice_from_values(a), dev.slice_from_values(b)
    dst = dev.allocate_uninit(DType.F32, n)
    dev.add(sa, sb, dst, n)
    dev.synchronize()
    assert np.array_equal(dst.to_vec(), oracle.gen_add(a, b))     # one rounded add: exact
    dev.silu_mul(sa, sb, dst, n)
    dev.synchronize()
    assert rel_err(dst.to_vec(), oracle.gen_silu_mul(a, b), 1e-20) < 1e-5
