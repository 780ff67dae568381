"""The allocation-free decode attention entry point against the ordinary one.

Some users of the library may not allocate GPU memory after start-up (their
process has handed the whole device to its own pool, or the calling thread
must never wait on an allocator), so ``ugb_decode_attention_noalloc`` works
out of a fixed scratch array inside the library.  The array is shared by all
calls and keeps the previous call's contents, so this test makes two calls in
a row with different shapes and compares each with ``ugb_decode_attention``
on the same inputs.  Both entry points run the same kernel in the same launch
shape, so the outputs must be equal bit for bit (and, a fortiori, within the
2e-2 tolerance the other attention tests use).
Collected last on purpose: a failure here stops nothing else.
"""
import ctypes as C

import numpy as np
import pytest

import oracle
from ug_b200 import DType, UgError, synth
from ug_b200._lib import lib

pytestmark = pytest.mark.gpu


def _inputs(dev, b, nh, nkv, t_max, seed):
    q = oracle.round_bf16(synth.normal(seed, (b, nh, 64)))
    k = oracle.round_bf16(synth.normal(seed + 1, (b, nkv, t_max, 64)))
    v = oracle.round_bf16(synth.normal(seed + 2, (b, nkv, t_max, 64)))
    return tuple(dev.slice_from_values(synth.to_bf16_bits(a), bf16=True) for a in (q, k, v))


def _run(dev, fn, sq, sk, sv, T, b, nh, nkv, t_max, slices):
    pos = dev.slice_from_values(np.array([T - 1], np.int32))
    out = dev.allocate_uninit(DType.BF16, b * nh * 64)
    dev._check(fn(dev._h, sq._h, sk._h, sv._h, pos._h, out._h, b, nh, nkv, t_max, slices))
    dev.synchronize()
    return synth.bf16_bits_to_f32(out.to_vec()).reshape(b, nh * 64)


def test_noalloc_matches_allocating_entry_point_twice_in_a_row(dev):
    # first call: deep cache, 4 slices; second call: other shape, fewer slices, so stale
    # partial results and counters of the first call are still in the shared array
    cases = [(4, 32, 4, 512, 500, 4, 1300), (2, 8, 2, 64, 17, 2, 1310)]
    prepared = [(_inputs(dev, b, nh, nkv, t_max, seed), (T, b, nh, nkv, t_max, slices))
                for b, nh, nkv, t_max, T, slices, seed in cases]
    want = [_run(dev, lib.ugb_decode_attention, *inp, *args) for inp, args in prepared]
    got = [_run(dev, lib.ugb_decode_attention_noalloc, *inp, *args) for inp, args in prepared]
    for g, w in zip(got, want):
        assert np.all(np.isfinite(g))
        assert np.max(np.abs(g - w)) <= 2e-2 * np.abs(w).max()
        assert np.array_equal(g, w)


def test_noalloc_rejects_more_than_its_fixed_scratch(dev):
    b, nh, nkv, t_max = 65, 32, 4, 16           # 65 * 4 * 8 slices = 2080 slots > 2048
    sq, sk, sv = _inputs(dev, b, nh, nkv, t_max, 1320)
    pos = dev.slice_from_values(np.array([0], np.int32))
    out = dev.allocate_uninit(DType.BF16, b * nh * 64)
    rc = lib.ugb_decode_attention_noalloc(dev._h, sq._h, sk._h, sv._h, pos._h, out._h, b, nh, nkv, t_max, 8)
    assert rc == 3
    assert b"exceeds the fixed scratch" in lib.ugb_last_error(dev._h)
    with pytest.raises(UgError):
        dev._check(rc)
