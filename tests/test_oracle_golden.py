"""Pins the CPU oracle against the reference's own known-answer vectors
(ug-core/tests/basic_tests.rs, ug-core/src/common_tests.rs) and against
independent float64 computations.  CPU only."""
import json
import os

import numpy as np

import oracle
from conftest import rel_err

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
REF = json.load(open(os.path.join(GOLDEN, "reference_vectors.json")))

# ug-core/tests/basic_tests.rs:41-61 (same vector in :63-116 for the SSA forms)
SOFTMAX_IN = np.array(REF["softmax_2x4"]["input"], dtype=np.float32)
SOFTMAX_OUT = np.array(REF["softmax_2x4"]["output"], dtype=np.float32)


def test_custom_softmax_golden_bit_exact():
    assert np.array_equal(oracle.custom_softmax(SOFTMAX_IN).ravel(), SOFTMAX_OUT)


def test_generated_softmax_golden():
    # -ffast-math build: within an ulp or two of the interpreter's vector
    assert rel_err(oracle.gen_softmax(SOFTMAX_IN).ravel(), SOFTMAX_OUT) < 3e-7


def test_mm_golden():
    # ug-core/src/common_tests.rs:15-22: ones[4,2] . twos[2,3] = 4.0
    lhs = np.full((4, 2), 1.0, np.float32)
    rhs = np.full((2, 3), 2.0, np.float32)
    assert np.array_equal(oracle.matmul(lhs, rhs), np.full((4, 3), 4.0, np.float32))


def test_add_golden():
    # ug-core/src/common_tests.rs:6-13: 40 + 2 on a (5, 2) buffer
    out = oracle.gen_add(np.full((5, 2), 40.0, np.float32), np.full((5, 2), 2.0, np.float32))
    assert np.array_equal(out, np.full((5, 2), 42.0, np.float32))


def test_cat_outer_axis_golden():
    # ug-core/src/common_tests.rs:24-30 (axis 0 is the case ug-llama's cat also covers)
    a0 = np.array([[1., 2.], [3., 4.]], np.float32)
    a1 = a0 + np.float32(0.1)
    a1 = np.array([[1.1, 2.1], [3.1, 4.1]], np.float32)
    a2 = np.array([[1.2, 2.2], [3.2, 4.2]], np.float32)
    out = oracle.cat(oracle.cat(a0, a1, 0), a2, 0)
    assert np.array_equal(out.ravel(), np.array(
        [1.0, 2.0, 3.0, 4.0, 1.1, 2.1, 3.1, 4.1, 1.2, 2.2, 3.2, 4.2], np.float32))


def test_softmax_forms_agree_and_match_float64():
    x = np.random.default_rng(0).standard_normal((16, 257)).astype(np.float32) * 2
    x64 = x.astype(np.float64)
    e = np.exp(x64 - x64.max(-1, keepdims=True))
    ref = e / e.sum(-1, keepdims=True)
    assert rel_err(oracle.custom_softmax(x), ref) < 2e-6
    assert rel_err(oracle.gen_softmax(x), ref) < 5e-6


def test_rms_forms_match_float64():
    rng = np.random.default_rng(1)
    x = rng.standard_normal((8, 320)).astype(np.float32)
    g = rng.standard_normal((8, 320)).astype(np.float32)
    w = rng.uniform(0.5, 1.5, 320).astype(np.float32)
    x64 = x.astype(np.float64)
    rms = x64 / np.sqrt((x64 ** 2).mean(-1, keepdims=True) + 1e-5) * w
    assert rel_err(oracle.gen_rms_norm(x, w, 1e-5), rms, 1e-6) < 2e-6
    silu = g.astype(np.float64) / (1 + np.exp(-g.astype(np.float64)))
    assert rel_err(oracle.gen_rms_norm_silu_gate(x, w, g, 1e-5), rms * silu, 1e-6) < 5e-6
    assert rel_err(oracle.gen_silu_mul(g, x), silu * x64, 1e-6) < 2e-6


def _rope_tables(max_pos, d, theta=10000.0):
    # ug-llama/src/model.rs:278-295
    inv = np.array([1.0 / theta ** (i / d) for i in range(0, d, 2)], dtype=np.float32)
    ang = np.arange(max_pos, dtype=np.float32)[:, None] * inv[None, :]
    return np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)


def test_rope_matches_float64_and_is_a_rotation():
    rng = np.random.default_rng(2)
    b, h, t, d = 2, 3, 5, 16
    x = rng.standard_normal((b, h, t, d)).astype(np.float32)
    cos, sin = _rope_tables(32, d)
    pos = np.array([[7]], np.int32)
    y = oracle.rope(x, cos, sin, pos)
    c = cos[7:7 + t].astype(np.float64)[None, None]
    s = sin[7:7 + t].astype(np.float64)[None, None]
    x1, x2 = x[..., :d // 2].astype(np.float64), x[..., d // 2:].astype(np.float64)
    ref = np.concatenate([x1 * c - x2 * s, x1 * s + x2 * c], -1)
    assert np.max(np.abs(y - ref)) < 1e-6  # absolute: the difference of products cancels
    yi = oracle.rope_i(x, cos, sin, pos)
    xe, xo = x[..., 0::2].astype(np.float64), x[..., 1::2].astype(np.float64)
    refi = np.empty_like(ref)
    refi[..., 0::2] = xe * c - xo * s
    refi[..., 1::2] = xe * s + xo * c
    assert np.max(np.abs(yi - refi)) < 1e-6
    # rotations keep the norm of every head vector
    assert np.allclose(np.linalg.norm(y, axis=-1), np.linalg.norm(x, axis=-1), rtol=1e-5)


def test_causal_mask_and_index_select():
    x = np.arange(2 * 1 * 3 * 4, dtype=np.float32).reshape(2, 1, 3, 4)
    y = oracle.causal_mask(x)
    keep = np.tril(np.ones((3, 4), bool))
    assert np.array_equal(y[..., keep], x[..., keep])
    assert np.all(np.isneginf(y[..., ~keep]))
    emb = np.random.default_rng(3).standard_normal((10, 6)).astype(np.float32)
    ids = np.array([[3, 9, 0], [1, 1, 7]], np.int32)
    assert np.array_equal(oracle.index_select(emb, ids), emb[ids])


def test_bf16_rounding_matches_torch():
    import torch
    x = np.random.default_rng(4).standard_normal(4096).astype(np.float32) * 3
    x[:4] = [0.0, -0.0, 1.0039062, 65504.0]
    want = torch.from_numpy(x).bfloat16().float().numpy()
    assert np.array_equal(oracle.round_bf16(x), want)
    from ug_b200 import synth
    assert np.array_equal(synth.bf16_bits_to_f32(synth.to_bf16_bits(x)), want)
    assert np.array_equal(oracle.to_bf16_bits(x), synth.to_bf16_bits(x))


def test_gemm_standin_matches_float64():
    rng = np.random.default_rng(5)
    a = rng.standard_normal((3, 17, 33)).astype(np.float32)
    b = rng.standard_normal((3, 33, 9)).astype(np.float32)
    ref = a.astype(np.float64) @ b.astype(np.float64)
    assert np.max(np.abs(oracle.matmul(a, b) - ref)) < 1e-4
    bt = np.ascontiguousarray(b.transpose(0, 2, 1))
    assert np.max(np.abs(oracle.matmul(a, bt, transpose_rhs=True) - ref)) < 1e-4
    w = rng.standard_normal((9, 33)).astype(np.float32)  # shared [n, k] weight
    ref2 = a.astype(np.float64) @ w.astype(np.float64).T
    assert np.max(np.abs(oracle.matmul(a, w, transpose_rhs=True) - ref2)) < 1e-4


def test_oracle_reproduces_committed_fixtures():
    """tests/golden/oracle_fixtures.npz (written by tests/golden/make_fixtures.py): the Rust-semantics operators
    bit for bit; the emitted-C forms (gcc -ffast-math -march=native, CPU dependent) and the model to 1e-6."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("make_fixtures", os.path.join(GOLDEN, "make_fixtures.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    now = mod.build()
    fix = np.load(os.path.join(GOLDEN, "oracle_fixtures.npz"))
    assert set(fix.files) == set(now)
    for k in ("softmax_out", "rope_out", "rope_i_out", "llama_prompt", "softmax_in_seed"):
        assert np.array_equal(fix[k], now[k]), k
    assert rel_err(now["rms_silu_out"], fix["rms_silu_out"]) < 1e-6
    assert np.max(np.abs(now["llama_logits"] - fix["llama_logits"])) < 1e-5 * np.abs(fix["llama_logits"]).max()
