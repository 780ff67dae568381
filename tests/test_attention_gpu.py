"""GPU parity of the stand-alone decode attention entry point against the
reference operator chain (repeat, q.kT, scale, softmax, .v, head merge of
ug-llama/src/model.rs:231-245) evaluated by the CPU oracle on the same
bf16-rounded inputs.  Tolerance 2e-2 relative to the largest output (bf16
probabilities and bf16 output)."""
import numpy as np
import pytest

import oracle
from ug_b200 import DType, UgError, synth

pytestmark = pytest.mark.gpu


def reference_attention(q, k, v, T):
    """q [b, nh, 64]; k, v [b, nkv, t_max, 64] (f32 values of bf16 data); attends positions < T."""
    b, nh, d = q.shape
    nkv = k.shape[1]
    out = np.empty((b, nh * d), np.float32)
    for i in range(b):
        kr = np.ascontiguousarray(np.repeat(k[i, :, :T], nh // nkv, axis=0))       # model.rs:80-92
        vr = np.ascontiguousarray(np.repeat(v[i, :, :T], nh // nkv, axis=0))
        att = oracle.matmul(np.ascontiguousarray(q[i][:, None, :]), kr, transpose_rhs=True)   # [nh, 1, T]
        att = (att * np.float32(0.125)).astype(np.float32)
        att = oracle.custom_softmax(att)
        out[i] = oracle.matmul(att, vr).transpose(1, 0, 2).reshape(-1)
    return out


def setup_case(dev, b, nh, nkv, t_max, seed):
    q = oracle.round_bf16(synth.normal(seed, (b, nh, 64)))
    k = oracle.round_bf16(synth.normal(seed + 1, (b, nkv, t_max, 64)))
    v = oracle.round_bf16(synth.normal(seed + 2, (b, nkv, t_max, 64)))
    sq, sk, sv = (dev.slice_from_values(synth.to_bf16_bits(a), bf16=True) for a in (q, k, v))
    return q, k, v, sq, sk, sv


@pytest.mark.parametrize("b,nh,nkv,t_max,T,slices", [
    (2, 32, 4, 2176, 2049, 2),      # the benchmark's cache depth
    (3, 8, 1, 64, 1, 2),            # a single cached position, an empty second slice
    (2, 8, 2, 64, 16, 1), (2, 8, 2, 64, 17, 3), (1, 4, 4, 48, 33, 2),
    (1, 16, 2, 1024, 1000, 8), (5, 2, 1, 320, 300, 4)])
def test_decode_attention_matches_oracle(dev, b, nh, nkv, t_max, T, slices):
    q, k, v, sq, sk, sv = setup_case(dev, b, nh, nkv, t_max, 1100 + T)
    pos = dev.slice_from_values(np.array([T - 1], np.int32))
    out = dev.allocate_uninit(DType.BF16, b * nh * 64)
    dev.decode_attention(sq, sk, sv, pos, out, b, nh, nkv, t_max, slices)
    dev.synchronize()
    got = synth.bf16_bits_to_f32(out.to_vec()).reshape(b, nh * 64)
    ref = reference_attention(q, k, v, T)
    assert np.max(np.abs(got - ref)) < 2e-2 * np.abs(ref).max()


def test_decode_attention_of_one_hot_scores_copies_a_value_row(dev):
    """A query that matches exactly one key with a huge margin returns that key's value row:
    softmax -> one-hot, so the output is a bit-exact copy of bf16 data."""
    b, nh, nkv, t_max, T = 1, 8, 1, 64, 40
    k = np.zeros((b, nkv, t_max, 64), np.float32)
    k[0, 0, 23, :] = 8.0
    v = oracle.round_bf16(synth.normal(1201, (b, nkv, t_max, 64)))
    q = np.full((b, nh, 64), 8.0, np.float32)
    sq, sk, sv = (dev.slice_from_values(synth.to_bf16_bits(a), bf16=True) for a in (q, k, v))
    pos = dev.slice_from_values(np.array([T - 1], np.int32))
    out = dev.allocate_uninit(DType.BF16, b * nh * 64)
    dev.decode_attention(sq, sk, sv, pos, out, b, nh, nkv, t_max, 2)
    dev.synchronize()
    got = synth.bf16_bits_to_f32(out.to_vec()).reshape(nh, 64)
    assert np.array_equal(got, np.broadcast_to(v[0, 0, 23], (nh, 64)))


def test_decode_attention_errors(dev):
    s = dev.allocate_uninit(DType.BF16, 8 * 64 * 64)
    f = dev.allocate_uninit(DType.F32, 8 * 64 * 64)
    p = dev.allocate_uninit(DType.I32, 1)
    with pytest.raises(UgError) as e:
        dev.decode_attention(f, s, s, p, s, 1, 8, 1, 64, 2)
    assert e.value.code == 2
    with pytest.raises(UgError) as e:
        dev.decode_attention(s, s, s, p, s, 1, 8, 1, 40, 2)       # cache depth not a multiple of 16
    assert e.value.code == 3
    with pytest.raises(UgError) as e:
        dev.decode_attention(s, s, s, p, s, 1, 18, 2, 64, 2)      # 9 query heads per KV head
    assert e.value.code == 6
    with pytest.raises(UgError) as e:
        dev.decode_attention(s, s, s, p, s, 1, 8, 1, 64, 9)
    assert e.value.code == 1


# ---- causal attention for a block of new positions (Attention::fwd with seq_len > 1) -------------------------

def reference_causal_attention(q, k, v, pos0, seqs):
    """The reference operator chain (model.rs:231-245: repeat, q.kT, scale, causal_mask, softmax, .v, head merge)
    on q [b, t, nh, 64] and caches [b, nkv, t_max, 64].  With pos0 = 0 the mask is the reference's own
    (cpu_ops.rs:33-56, the block starts at key 0); for a block that continues a cache it is the same rule shifted
    by the cached positions (query i sees keys 0 .. pos0 + i), which the reference does not implement."""
    b, t, nh, d = q.shape
    nkv = k.shape[1]
    T = pos0 + t
    out = {}
    for i in seqs:
        kr = np.ascontiguousarray(np.repeat(k[i, :, :T], nh // nkv, axis=0))
        vr = np.ascontiguousarray(np.repeat(v[i, :, :T], nh // nkv, axis=0))
        qi = np.ascontiguousarray(q[i].transpose(1, 0, 2))                        # [nh, t, 64]
        att = (oracle.matmul(qi, kr, transpose_rhs=True) * np.float32(0.125)).astype(np.float32)   # [nh, t, T]
        if pos0 == 0:
            att = oracle.causal_mask(att[None])[0]
        else:
            att[:, np.arange(T)[None, :] > (pos0 + np.arange(t))[:, None]] = -np.inf
        att = oracle.custom_softmax(att)
        out[i] = oracle.matmul(att, vr).transpose(1, 0, 2).reshape(t, nh * d)
    return out


def causal_case(dev, b, nh, nkv, t, pos0, t_max, seed):
    q = oracle.round_bf16(synth.normal(seed, (b, t, nh, 64)))
    k = oracle.round_bf16(synth.normal(seed + 1, (b, nkv, t_max, 64)))
    v = oracle.round_bf16(synth.normal(seed + 2, (b, nkv, t_max, 64)))
    sq, sk, sv = (dev.slice_from_values(synth.to_bf16_bits(a), bf16=True) for a in (q, k, v))
    return q, k, v, sq, sk, sv


@pytest.mark.parametrize("b,nh,nkv,t,pos0,t_max", [
    (2, 8, 2, 100, 0, 128),        # ragged last query tile
    (1, 4, 4, 1, 0, 64),           # a block of one position
    (3, 16, 2, 64, 37, 128),       # continues a cache; the block starts inside a key tile
    (2, 12, 4, 200, 0, 256),       # three query heads per KV head
    (2, 9, 1, 70, 5, 80),          # nine query heads per KV head; the last key tile runs past the cache's end
    (4, 32, 4, 1280, 0, 1280),     # 1280 work items of 2 to 20 key tiles on 296 persistent CTAs
])
def test_causal_attention_matches_oracle(dev, b, nh, nkv, t, pos0, t_max):
    q, k, v, sq, sk, sv = causal_case(dev, b, nh, nkv, t, pos0, t_max, 1300 + t)
    out = dev.allocate_uninit(DType.BF16, b * t * nh * 64)
    dev.causal_attention(sq, sk, sv, out, b, t, pos0, nh, nkv, t_max)
    dev.synchronize()
    got = synth.bf16_bits_to_f32(out.to_vec()).reshape(b, t, nh * 64)
    seqs = sorted({0, b - 1})
    ref = reference_causal_attention(q, k, v, pos0, seqs)
    for i in seqs:
        assert np.max(np.abs(got[i] - ref[i])) < 2e-2 * np.abs(ref[i]).max()
    # the same call again gives the same bits (the work counter is back at zero after a launch)
    dev.causal_attention(sq, sk, sv, out, b, t, pos0, nh, nkv, t_max)
    dev.synchronize()
    assert np.array_equal(synth.bf16_bits_to_f32(out.to_vec()).reshape(b, t, nh * 64), got)


def test_causal_attention_of_one_hot_scores_copies_a_value_row(dev):
    """Queries at and after position 23 match key 23 with a huge margin: their softmax is one-hot and the output
    a bit-exact copy of that bf16 value row; the queries before it average the value rows they see."""
    b, nh, nkv, t, t_max = 1, 8, 1, 90, 128
    k = np.zeros((b, nkv, t_max, 64), np.float32)
    k[0, 0, 23, :] = 8.0
    v = oracle.round_bf16(synth.normal(1401, (b, nkv, t_max, 64)))
    q = np.full((b, t, nh, 64), 8.0, np.float32)
    sq, sk, sv = (dev.slice_from_values(synth.to_bf16_bits(a), bf16=True) for a in (q, k, v))
    out = dev.allocate_uninit(DType.BF16, b * t * nh * 64)
    dev.causal_attention(sq, sk, sv, out, b, t, 0, nh, nkv, t_max)
    dev.synchronize()
    got = synth.bf16_bits_to_f32(out.to_vec()).reshape(t, nh, 64)
    assert np.array_equal(got[23:], np.broadcast_to(v[0, 0, 23], (t - 23, nh, 64)))
    for i in (0, 7, 22):
        want = v[0, 0, :i + 1].mean(axis=0)
        assert np.max(np.abs(got[i] - want[None, :])) <= 2.0 ** -8 * np.abs(want).max() + 1e-6


def test_causal_attention_errors(dev):
    s = dev.allocate_uninit(DType.BF16, 8 * 64 * 64)
    f = dev.allocate_uninit(DType.F32, 8 * 64 * 64)
    with pytest.raises(UgError) as e:
        dev.causal_attention(f, s, s, s, 1, 8, 0, 8, 1, 64)
    assert e.value.code == 2
    with pytest.raises(UgError) as e:
        dev.causal_attention(s, s, s, s, 1, 8, 60, 8, 1, 64)      # positions 60..68 in a cache of 64
    assert e.value.code == 3
    with pytest.raises(UgError) as e:
        dev.causal_attention(s, s, s, s, 1, 8, 0, 9, 2, 64)       # 9 query heads over 2 KV heads
    assert e.value.code == 6
    with pytest.raises(UgError) as e:
        dev.causal_attention(s, s, s, s, 4, 64, 0, 8, 1, 64)      # q shorter than b * t * n_heads * 64
    assert e.value.code == 3
    dev.causal_attention(s, s, s, s, 0, 8, 0, 8, 1, 64)           # an empty batch is a no-op
