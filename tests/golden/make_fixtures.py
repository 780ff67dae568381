"""Writes tests/golden/oracle_fixtures.npz: outputs of the CPU oracle on seeded inputs.

The reference itself cannot be run in this environment (Rust, no toolchain), so these are not reference
outputs: they freeze what the oracle -- pinned against the reference's own known-answer vectors in
reference_vectors.json -- computes, so that a change of the oracle, of the synthetic generator or of a
kernel shows up against a committed file.  Run from the repository root:  python tests/golden/make_fixtures.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)


def build():
    import oracle
    from oracle import llama_ref as R
    from ug_b200 import synth
    from ug_b200.llama import Config

    out = {}
    x = synth.normal(0, (4, 33), 2.0)
    out["softmax_in_seed"] = np.array([0, 4, 33], np.int64)
    out["softmax_out"] = oracle.custom_softmax(x)
    q = synth.normal(41, (1, 2, 5, 64))
    cos = np.cos(np.arange(16 * 32, dtype=np.float32).reshape(16, 32) * np.float32(0.01)).astype(np.float32)
    sin = np.sin(np.arange(16 * 32, dtype=np.float32).reshape(16, 32) * np.float32(0.01)).astype(np.float32)
    pos = np.array([[3]], np.int32)
    out["rope_out"] = oracle.rope(q, cos, sin, pos)
    out["rope_i_out"] = oracle.rope_i(q, cos, sin, pos)
    xg, g = synth.normal(42, (6, 128)), synth.normal(43, (6, 128))
    w = synth.uniform(44, (128,), 0.5, 1.5)
    out["rms_silu_out"] = oracle.gen_rms_norm_silu_gate(xg, w, g, 1e-5)
    cfg = Config(hidden_size=128, intermediate_size=256, max_position_embeddings=64, num_attention_heads=2,
                 num_key_value_heads=1, num_hidden_layers=2, vocab_size=512)
    weights = synth.llama_weights(cfg, 100)
    ref = R.Model(R.Config(**cfg.__dict__), synth.llama_weights_f32(weights))
    prompts = synth.tokens(7, (1, 12), cfg.vocab_size)
    out["llama_prompt"] = prompts
    out["llama_logits"] = ref.fwd(prompts, 0, ref.new_cache())[0]
    return out


if __name__ == "__main__":
    np.savez_compressed(os.path.join(ROOT, "tests", "golden", "oracle_fixtures.npz"), **build())
    print("written", os.path.join("tests", "golden", "oracle_fixtures.npz"))
