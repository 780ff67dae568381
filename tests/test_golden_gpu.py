"""CUDA path against the committed fixtures of tests/golden/ (through the C ABI): the reference's own
known-answer vectors, and the frozen oracle outputs on seeded inputs."""
import json
import os

import numpy as np
import pytest

from conftest import rel_err
from ug_b200 import DType, synth
from ug_b200.llama import Config, Model

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
REF = json.load(open(os.path.join(GOLDEN, "reference_vectors.json")))
FIX = np.load(os.path.join(GOLDEN, "oracle_fixtures.npz"))


def test_reference_softmax_vector(dev):
    x = np.array(REF["softmax_2x4"]["input"], np.float32)
    src, dst = dev.slice_from_values(x), dev.allocate_uninit(DType.F32, x.size)
    dev.custom_softmax(src, dst, 2, 4)
    dev.synchronize()
    assert rel_err(dst.to_vec(), np.array(REF["softmax_2x4"]["output"], np.float32)) < 1e-6   # fp32 reduction: <= 1e-5


def test_reference_mm_vector(dev):
    g = REF["mm_ones_twos"]
    (m, k), (_, n) = g["lhs_shape"], g["rhs_shape"]
    a = dev.slice_from_values(np.full((m, k), g["lhs_value"], np.float32))
    b = dev.slice_from_values(np.full((k, n), g["rhs_value"], np.float32))
    c = dev.allocate_uninit(DType.F32, m * n)
    dev.matmul(c, a, b, (1, m, n, k), ([1, m, k], [m * k, k, 1], 0), ([1, k, n], [k * n, n, 1], 0))
    dev.synchronize()
    assert np.array_equal(c.to_vec(), np.full(m * n, g["output_value"], np.float32))


def test_frozen_softmax_rope_and_rms_silu(dev):
    x = synth.normal(0, (4, 33), 2.0)
    src, dst = dev.slice_from_values(x), dev.allocate_uninit(DType.F32, x.size)
    dev.custom_softmax(src, dst, 4, 33)
    q = synth.normal(41, (1, 2, 5, 64))
    cos = np.cos(np.arange(16 * 32, dtype=np.float32).reshape(16, 32) * np.float32(0.01)).astype(np.float32)
    sin = np.sin(np.arange(16 * 32, dtype=np.float32).reshape(16, 32) * np.float32(0.01)).astype(np.float32)
    qs, cs, ss = (dev.slice_from_values(a) for a in (q, cos, sin))
    ps = dev.slice_from_values(np.array([3], np.int32))
    r, ri = dev.allocate_uninit(DType.F32, q.size), dev.allocate_uninit(DType.F32, q.size)
    dev.rope(qs, cs, ss, ps, r, 1, 2, 5, 64)
    dev.rope_i(qs, cs, ss, ps, ri, 1, 2, 5, 64)
    xg, g = synth.normal(42, (6, 128)), synth.normal(43, (6, 128))
    w = synth.uniform(44, (128,), 0.5, 1.5)
    out = dev.allocate_uninit(DType.F32, xg.size)
    dev.rms_norm_silu_gate(dev.slice_from_values(xg), dev.slice_from_values(w), dev.slice_from_values(g), out, 6, 128, 1e-5)
    dev.synchronize()
    assert rel_err(dst.to_vec().reshape(4, 33), FIX["softmax_out"]) < 1e-5
    assert np.array_equal(r.to_vec().reshape(q.shape), FIX["rope_out"])          # separately rounded products: bit-exact
    assert np.array_equal(ri.to_vec().reshape(q.shape), FIX["rope_i_out"])
    assert rel_err(out.to_vec().reshape(6, 128), FIX["rms_silu_out"]) < 1e-5


def test_frozen_llama_logits(dev):
    cfg = Config(hidden_size=128, intermediate_size=256, max_position_embeddings=64, num_attention_heads=2,
                 num_key_value_heads=1, num_hidden_layers=2, vocab_size=512)
    prompts = FIX["llama_prompt"]
    assert np.array_equal(prompts, synth.tokens(7, (1, 12), cfg.vocab_size))
    m = Model.new(cfg, synth.llama_weights(cfg, 100), dev, 1, 32)
    m.prefill(prompts, all_logits=True)
    got = m.prefill_logits()[0]
    want = FIX["llama_logits"]
    assert np.max(np.abs(got - want)) < 2e-2 * np.abs(want).max()
    m.reset(0)
    for i in range(prompts.shape[1]):      # the same positions one token at a time
        m.fwd(prompts[:, i])
        assert np.max(np.abs(m.logits()[0] - want[i])) < 2e-2 * np.abs(want).max()
    m.close()
