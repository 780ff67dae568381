"""Error paths that end in a status code instead of a fault or a hang, through the C ABI.

* A device-side wait whose limit runs out (nothing ever completes what it waits for) makes the kernel
  return and the next ugb_sync report UGB_ERR_TIMEOUT (7) with the site code; the device handle works
  afterwards.  The wait gives up by design: nothing faults, nothing hangs.
* A device-side position that points outside the KV cache or the rope tables makes the stand-alone
  operators skip all accesses and raise UGB_ERR_INVALID (1), where the reference panics on a slice bound.
"""
import time

import numpy as np
import pytest

import oracle
from ug_b200 import DType, UgError, synth
from ug_b200._lib import lib

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("which,site", [(0, 0x99), (1, 0x7001)])
def test_bounded_wait_runs_out_and_reports_timeout(dev, which, site):
    dev.synchronize()
    dev.set_option("wait_limit_us", 2000)                 # 2 ms
    try:
        t0 = time.perf_counter()
        dev._check(lib.ugb_selftest_bounded_wait(dev._h, which))
        with pytest.raises(UgError) as e:
            dev.synchronize()
        waited = time.perf_counter() - t0
        assert e.value.code == 7
        assert f"detail {site}" in str(e.value)
        assert waited < 1.0                               # the 2 ms limit, not the 2 s default
    finally:
        dev.set_option("wait_limit_us", 2000000)
    # the status word was cleared by the failing sync; the handle is as usable as before
    dev.synchronize()
    x = synth.normal(5, (4, 256))
    sx = dev.slice_from_values(x)
    out = dev.allocate_uninit(DType.F32, x.size)
    dev.custom_softmax(sx, out, 4, 256)
    dev.synchronize()
    ref = oracle.custom_softmax(x)
    assert np.max(np.abs(out.to_vec().reshape(4, 256) - ref) / ref) < 1e-5


def test_wait_limit_option_range(dev):
    for bad in (0, 99, 60000001):
        with pytest.raises(UgError):
            dev.set_option("wait_limit_us", bad)


@pytest.mark.parametrize("bad_pos", [64, 100000, -5])
def test_decode_attention_rejects_a_position_outside_the_cache(dev, bad_pos):
    b, nh, nkv, t_max = 2, 8, 2, 64
    q = synth.to_bf16_bits(synth.normal(1, (b, nh, 64)))
    kv = synth.to_bf16_bits(synth.normal(2, (b, nkv, t_max, 64)))
    sq, sk, sv = (dev.slice_from_values(a, bf16=True) for a in (q, kv, kv))
    pos = dev.slice_from_values(np.array([bad_pos], np.int32))
    sentinel = np.full(b * nh * 64, 0x7FC0, np.uint16)    # bf16 NaN pattern: "untouched"
    out = dev.slice_from_values(sentinel, bf16=True)
    dev.decode_attention(sq, sk, sv, pos, out, b, nh, nkv, t_max, 2)
    with pytest.raises(UgError) as e:
        dev.synchronize()
    assert e.value.code == 1
    assert np.array_equal(out.to_vec(), sentinel)
    # the largest legal position still works
    pos_ok = dev.slice_from_values(np.array([t_max - 1], np.int32))
    dev.decode_attention(sq, sk, sv, pos_ok, out, b, nh, nkv, t_max, 2)
    dev.synchronize()
    assert not np.array_equal(out.to_vec(), sentinel)


@pytest.mark.parametrize("interleaved", [False, True])
def test_rope_rejects_a_position_outside_the_tables(dev, interleaved):
    b, h, t, d, max_pos = 1, 2, 3, 64, 16
    x = synth.normal(3, (b, h, t, d))
    cos, sin = synth.normal(4, (max_pos, d // 2)), synth.normal(5, (max_pos, d // 2))
    sx, sc, ss = (dev.slice_from_values(a) for a in (x, cos, sin))
    op = dev.rope_i if interleaved else dev.rope
    sentinel = np.full(x.size, -7.0, np.float32)
    for bad in (max_pos - t + 1, 1 << 20, -1):
        out = dev.slice_from_values(sentinel)
        op(sx, sc, ss, dev.slice_from_values(np.array([bad], np.int32)), out, b, h, t, d)
        with pytest.raises(UgError) as e:
            dev.synchronize()
        assert e.value.code == 1
        assert np.array_equal(out.to_vec(), sentinel)
    out = dev.slice_from_values(sentinel)
    op(sx, sc, ss, dev.slice_from_values(np.array([max_pos - t], np.int32)), out, b, h, t, d)   # last legal start
    dev.synchronize()
    ref = (oracle.rope_i if interleaved else oracle.rope)(x, cos, sin, np.array([[max_pos - t]], np.int32))
    assert np.array_equal(out.to_vec().reshape(x.shape), ref)
