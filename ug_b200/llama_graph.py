"""ug-llama's model on the lazy graph: the operator wrappers of
ug-llama/src/cuda_ops.rs (rope, rope_i, cat, custom_softmax, causal_mask as
``LB::custom`` nodes, arguments in call order and the destination last) and
the graph construction of ug-llama/src/model.rs (index_select as hand-built
SSA, rms_norm, repeat, softmax, silu, Linear, Mlp, Attention, Layer, Rope,
Model), all f32 as in the reference.  ``Model.fwd`` builds the graph for any
seq_len and one sequence, exactly like the reference (batch 1)."""
import numpy as np

from .device import DType
from .lazy import LB, BinaryOp as B, ReduceOp as R, UnaryOp as U, ssa


# ------------------------------------------------ ug_llama::Device operators
def custom_softmax(src):
    dims = src.dims()
    n_cols = dims[-1]
    n_rows = int(np.prod(dims, dtype=np.int64)) // n_cols
    ops = src.device.ops
    return LB.custom(lambda s: ops.softmax(s[0], s[1], n_rows, n_cols), [src], dims, src.dtype(), src.device)


def causal_mask(src):
    b, h, s1, s2 = src.dims()
    ops = src.device.ops
    return LB.custom(lambda s: ops.causal_mask(s[0], s[1], b * h, s1, s2), [src], src.dims(), src.dtype(), src.device)


def _rope(interleaved, src, cos, sin, pos):
    b, h, t, d = src.dims()
    ops = src.device.ops
    return LB.custom(lambda s: ops.rope(interleaved, s[0], s[1], s[2], s[3], s[4], b, h, t, d),
                     [src, cos, sin, pos], (b, h, t, d), src.dtype(), src.device)


def rope(src, cos, sin, pos):
    return _rope(False, src, cos, sin, pos)


def rope_i(src, cos, sin, pos):
    return _rope(True, src, cos, sin, pos)


def cat(lhs, rhs, axis):
    l, r = lhs.dims(), rhs.dims()
    if axis >= len(l):
        raise ValueError(f"unexpected axis {axis} for cat {l}")
    if len(l) != len(r) or any(i != axis and a != b for i, (a, b) in enumerate(zip(l, r))):
        raise ValueError(f"unexpected shapes for cat {l} {r} axis: {axis}")
    dst = list(l)
    dst[axis] = l[axis] + r[axis]
    d1 = int(np.prod(l[:axis], dtype=np.int64))
    d2_l = int(np.prod(l[axis:], dtype=np.int64))
    d2_r = int(np.prod(r[axis:], dtype=np.int64))
    ops = lhs.device.ops
    return LB.custom(lambda s: ops.cat(s[0], s[1], s[2], d1, d2_l, d2_r), [lhs, rhs], dst, lhs.dtype(), lhs.device)


# --------------------------------------------------------------- model.rs ----
def index_select(src, ids):
    """model.rs:32-63: two nested Range loops in hand-built SSA; the id is loaded with dtype tag F32
    from the I32 buffer, as the reference does (model.rs:49)."""
    b_sz, seq_len = ids.dims()
    _, h = src.dims()
    f32, i32 = DType.F32, DType.I32
    I = ssa.instr
    ins = [
        I("DefineGlobal", f32, index=0),                                   # 0 src
        I("DefineGlobal", i32, index=1),                                   # 1 ids
        I("DefineGlobal", f32, index=2),                                   # 2 dst
        I("Range", a0=ssa.i32(0), a1=ssa.i32(b_sz * seq_len), index=1, v0=13),   # 3 r1
        I("Load", f32, v0=1, a0=3),                                        # 4 ids[r1] (as f32)
        I("Binary", i32, op=B.Mul, a0=4, a1=ssa.i32(h)),                   # 5 src_off
        I("Binary", i32, op=B.Mul, a0=3, a1=ssa.i32(h)),                   # 6 dst_off
        I("Range", a0=ssa.i32(0), a1=ssa.i32(h), index=1, v0=12),          # 7 r2
        I("Binary", i32, op=B.Add, a0=5, a1=7),                            # 8
        I("Binary", i32, op=B.Add, a0=6, a1=7),                            # 9
        I("Load", f32, v0=0, a0=8),                                        # 10
        I("Store", f32, v0=2, a0=9, a1=10),                                # 11
        I("EndRange", v0=7),                                               # 12
        I("EndRange", v0=3),                                               # 13
    ]
    return LB.ssa(ins, [src, ids], (b_sz, seq_len, h), src.dtype(), src.device)


def rms_norm(src, alpha, eps):
    """model.rs:65-78"""
    dev, s = src.device, src.dims()
    dim_m1 = s[-1]
    sum2 = src.binary(B.Mul, src).reduce(R.Sum, len(s) - 1)
    m = (sum2.binary(B.Mul, LB.cst(np.float32(1.0) / np.float32(dim_m1), s, dev))
         .binary(B.Add, LB.cst(np.float32(eps), s, dev)).unary(U.Sqrt))
    return src.binary(B.Div, m.broadcast(s)).binary(B.Mul, alpha.broadcast(s))


def repeat(lb, axis, n_rep):
    """model.rs:80-92"""
    if n_rep == 1:
        return lb
    dims = lb.dims()
    lb = lb.split_dim(axis, dims[axis], 1)
    d = list(lb.dims())
    d[axis + 1] = n_rep
    return lb.broadcast(d).merge_dims(axis)


def softmax(src):
    """model.rs:94-101"""
    s = src.dims()
    mx = src.reduce(R.Max, -1)
    diff = src.binary(B.Sub, mx.broadcast(s))
    e = diff.unary(U.Exp)
    return e.binary(B.Div, e.reduce(R.Sum, -1).broadcast(s))


def silu(src):
    """model.rs:103-109"""
    exp_m = src.unary(U.Neg).unary(U.Exp)
    one = LB.cst(1.0, (), src.device).broadcast(exp_m.dims())
    return src.binary(B.Div, exp_m.binary(B.Add, one))


class Model:
    """Model::new / Model::fwd (model.rs:298-374) over f32 weights (name -> numpy array)."""

    def __init__(self, cfg, weights, device, custom_softmax_op=False):
        self.cfg, self.dev, self.custom_softmax = cfg, device, custom_softmax_op
        self.w = {k: LB.copy(np.asarray(v, np.float32), v.shape, device) for k, v in weights.items()}
        hd = cfg.head_dim()
        theta = np.array([np.float32(1.0) / np.float32(cfg.rope_theta) ** (np.float32(i) / np.float32(hd))
                          for i in range(0, hd, 2)], np.float32)          # Rope::new, model.rs:278-295
        idx = np.arange(cfg.max_position_embeddings, dtype=np.float32)
        mm = LB.copy(idx, (cfg.max_position_embeddings, 1), device).matmul(LB.copy(theta, (1, hd // 2), device))
        self.cos, self.sin = mm.unary(U.Cos), mm.unary(U.Sin)

    def new_cache(self):
        c = self.cfg
        shape = (1, c.num_key_value_heads, 0, c.head_dim())
        return [[LB.cst(0.0, shape, self.dev), LB.cst(0.0, shape, self.dev)] for _ in range(c.num_hidden_layers)]

    def _attention(self, xs, i, pos, cache):
        c, p = self.cfg, f"model.layers.{i}.self_attn"
        nh, nkv, hd = c.num_attention_heads, c.num_key_value_heads, c.head_dim()
        _, seq_len, _ = xs.dims()
        q = xs.matmul_t(self.w[f"{p}.q_proj.weight"]).split_dim(2, nh, hd).transpose(2, 1)
        k = xs.matmul_t(self.w[f"{p}.k_proj.weight"]).split_dim(2, nkv, hd).transpose(2, 1)
        v = xs.matmul_t(self.w[f"{p}.v_proj.weight"]).split_dim(2, nkv, hd).transpose(2, 1)
        r = rope_i if c.rope_interleaved else rope
        q, k = r(q, self.cos, self.sin, pos), r(k, self.cos, self.sin, pos)
        k = cat(cache[i][0], k, 2)
        v = cat(cache[i][1], v, 2)
        cache[i][0], cache[i][1] = k, v
        k, v = repeat(k, 1, nh // nkv), repeat(v, 1, nh // nkv)
        att = q.matmul_t(k)
        scale = LB.cst(np.float32(hd) ** np.float32(-0.5), (), self.dev).broadcast(att.dims())
        att = att.binary(B.Mul, scale)
        if seq_len != 1:
            att = causal_mask(att)
        att = custom_softmax(att) if self.custom_softmax else softmax(att)
        xs = att.matmul(v).transpose(2, 1).merge_dims(-2)
        return xs.matmul_t(self.w[f"{p}.o_proj.weight"])

    def fwd(self, tokens, pos, cache):
        """tokens, pos: LazyBuffers (I32 [1, t] and [1, 1]); returns the logits node [1, t, vocab]."""
        c, eps = self.cfg, self.cfg.rms_norm_eps
        xs = index_select(self.w["model.embed_tokens.weight"], tokens)
        for i in range(c.num_hidden_layers):
            p = f"model.layers.{i}"
            residual = xs
            h = rms_norm(xs, self.w[f"{p}.input_layernorm.weight"], eps)
            xs = self._attention(h, i, pos, cache).binary(B.Add, residual)
            residual = xs
            h = rms_norm(xs, self.w[f"{p}.post_attention_layernorm.weight"], eps)
            g = silu(h.matmul_t(self.w[f"{p}.mlp.gate_proj.weight"]))
            u = h.matmul_t(self.w[f"{p}.mlp.up_proj.weight"])
            xs = g.binary(B.Mul, u).matmul_t(self.w[f"{p}.mlp.down_proj.weight"]).binary(B.Add, residual)
        xs = rms_norm(xs, self.w["model.norm.weight"], eps)
        return xs.matmul_t(self.w["model.embed_tokens.weight"])
