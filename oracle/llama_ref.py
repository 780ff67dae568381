"""CPU oracle of ug-llama's forward pass -- TEST INFRASTRUCTURE ONLY.

Follows ug-llama/src/model.rs operator by operator, in f32, for ONE sequence
at a time (the reference model only runs b_sz = 1: LazyBuffer::matmul_ needs
equal batch sizes, ug-core/src/lazy_buffer.rs:432-436, and Cache::new is
batch 1, model.rs:192-193).  A batch is a list of independent sequences.

Every arithmetic step goes through the C restatements of this directory:
emitted-C kernels for the lazy-graph ops (rms_norm, silu*up, softmax, add),
ug-llama's CPU custom ops (rope, cat, causal_mask, custom_softmax), and the
f32 GEMM stand-in for crate gemm.  Weights are f32 values that were rounded to
bf16 first, which is what load_with_cast BF16 -> F32 yields
(ug-core/src/safetensors.rs:153-157).

Parity status: ug-llama has no tests, so this file is "parity unpinned"
against the reference itself; it is pinned operator by operator through the
known-answer vectors and float64 cross-checks of tests/test_oracle_golden.py.
"""
import numpy as np

from . import (cat, causal_mask, custom_softmax, gen_add, gen_rms_norm, gen_silu_mul,
               gen_softmax, index_select, matmul, rope, rope_i)


class Config:
    """ug_llama::model::Config (model.rs:10-30)."""

    def __init__(self, hidden_size, intermediate_size, max_position_embeddings, num_attention_heads,
                 num_key_value_heads, num_hidden_layers, vocab_size, rms_norm_eps=1e-5,
                 rope_theta=10000.0, rope_interleaved=False, tie_word_embeddings=True):
        self.hidden_size = hidden_size
        self.intermediate_size = intermediate_size
        self.max_position_embeddings = max_position_embeddings
        self.num_attention_heads = num_attention_heads
        self.num_key_value_heads = num_key_value_heads
        self.num_hidden_layers = num_hidden_layers
        self.vocab_size = vocab_size
        self.rms_norm_eps = rms_norm_eps
        self.rope_theta = rope_theta
        self.rope_interleaved = rope_interleaved
        self.tie_word_embeddings = tie_word_embeddings

    def head_dim(self):
        return self.hidden_size // self.num_attention_heads


def rope_tables(cfg):
    """Rope::new (model.rs:278-295): theta in f32, outer product, cos / sin."""
    d = cfg.head_dim()
    theta = np.array([np.float32(1.0) / np.float32(cfg.rope_theta) ** (np.float32(i) / np.float32(d))
                      for i in range(0, d, 2)], dtype=np.float32)
    idx = np.arange(cfg.max_position_embeddings, dtype=np.float32)
    mm = (idx[:, None] * theta[None, :]).astype(np.float32)   # k = 1 matmul: single f32 products
    return np.cos(mm).astype(np.float32), np.sin(mm).astype(np.float32)


def repeat(x, axis, n_rep):
    """model.rs:80-92: split_dim -> broadcast -> merge_dims."""
    return x if n_rep == 1 else np.repeat(x, n_rep, axis=axis)


class Model:
    """Model::new / Model::fwd (model.rs:298-374) with Cache (model.rs:183-198)."""

    def __init__(self, cfg, weights, custom_softmax_op=True):
        if not cfg.tie_word_embeddings:
            raise ValueError("tie_word_embeddings == false is not supported yet")   # model.rs:318
        self.cfg = cfg
        self.w = weights
        self.cos, self.sin = rope_tables(cfg)
        self.custom_softmax = custom_softmax_op

    def new_cache(self):
        c = self.cfg
        z = np.zeros((1, c.num_key_value_heads, 0, c.head_dim()), np.float32)
        return [[z.copy(), z.copy()] for _ in range(c.num_hidden_layers)]

    def _linear(self, x, name):
        return matmul(x, self.w[name], transpose_rhs=True)     # Linear::fwd = matmul_t

    def _attention(self, xs, i, pos, cache):
        c, p = self.cfg, f"model.layers.{i}.self_attn"
        nh, nkv, hd = c.num_attention_heads, c.num_key_value_heads, c.head_dim()
        _, t, _ = xs.shape
        q = self._linear(xs, f"{p}.q_proj.weight").reshape(1, t, nh, hd).transpose(0, 2, 1, 3)
        k = self._linear(xs, f"{p}.k_proj.weight").reshape(1, t, nkv, hd).transpose(0, 2, 1, 3)
        v = self._linear(xs, f"{p}.v_proj.weight").reshape(1, t, nkv, hd).transpose(0, 2, 1, 3)
        q, k, v = (np.ascontiguousarray(a) for a in (q, k, v))
        r = rope_i if c.rope_interleaved else rope
        pos_a = np.array([[pos]], np.int32)
        q = r(q, self.cos, self.sin, pos_a)
        k = r(k, self.cos, self.sin, pos_a)
        k = cat(cache[i][0], k, 2)
        v = cat(cache[i][1], v, 2)
        cache[i][0], cache[i][1] = k, v
        kr = np.ascontiguousarray(repeat(k, 1, nh // nkv))[0]
        vr = np.ascontiguousarray(repeat(v, 1, nh // nkv))[0]
        att = matmul(q[0], kr, transpose_rhs=True)              # [nh, t, T]
        np.multiply(att, np.float32(np.float32(hd) ** np.float32(-0.5)), out=att)   # f32 * f32, in place
        att = att[None]
        if t != 1:
            att = causal_mask(att)
        att = custom_softmax(att) if self.custom_softmax else gen_softmax(att)
        o = matmul(att[0], vr)                                   # [nh, t, hd]
        o = np.ascontiguousarray(o.transpose(1, 0, 2)).reshape(1, t, nh * hd)
        return self._linear(o, f"{p}.o_proj.weight")

    def fwd(self, tokens, pos, cache):
        """tokens int32 [1, t]; returns logits f32 [1, t, vocab]."""
        c = self.cfg
        eps = np.float32(c.rms_norm_eps)
        xs = index_select(self.w["model.embed_tokens.weight"], tokens)
        for i in range(c.num_hidden_layers):
            p = f"model.layers.{i}"
            residual = xs
            h = gen_rms_norm(xs, self.w[f"{p}.input_layernorm.weight"], eps)
            h = self._attention(h, i, pos, cache)
            xs = gen_add(h, residual)
            residual = xs
            h = gen_rms_norm(xs, self.w[f"{p}.post_attention_layernorm.weight"], eps)
            g = self._linear(h, f"{p}.mlp.gate_proj.weight")
            u = self._linear(h, f"{p}.mlp.up_proj.weight")
            h = self._linear(gen_silu_mul(g, u), f"{p}.mlp.down_proj.weight")
            xs = gen_add(h, residual)
        xs = gen_rms_norm(xs, self.w["model.norm.weight"], eps)
        return self._linear(xs, "model.embed_tokens.weight")
