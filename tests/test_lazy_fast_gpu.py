"""Graph kernels on generated 128-bit code (host layer: ug_fast.cpp) on the B200 device: which generator each
item of a compiled schedule ran on, and parity with ug's CPU backend (the oracle's emitted-C kernels) within
1e-5 relative for fp32 reductions.  The unmodified graph forms of ug-llama/src/model.rs:65-109 are used."""
import numpy as np
import pytest

import oracle
import ug_b200
from ug_b200 import llama_graph as G
from ug_b200 import synth
from ug_b200.lazy import LB, BinaryOp as B, HostDevice, Schedule

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def hd(dev):
    return HostDevice(dev)


def run(y):
    s = Schedule.create_one(y)
    c = s.compile()
    c.run()
    return s, c, y.data_vec()


@pytest.mark.parametrize("rows,cols", [(8192, 4096), (33, 1024), (7, 32000), (130, 64), (3, 12), (5, 2100)])
def test_graph_softmax_is_one_row_kernel(hd, rows, cols):
    x = synth.normal(11, (rows, cols), 2.0)
    s, c, got = run(G.softmax(LB.copy(x, (rows, cols), hd)))
    # exp(x - max) feeds the sum and the division of the same row: evaluated in place, one kernel, one read, one write
    assert s.items() == ["Kernel"]
    expect = "warp_row_vec4" if cols <= 1024 else "row_vec4"
    assert c.origins() == [expect]
    check = min(rows, 48)
    ref = oracle.custom_softmax(x[:check])
    assert np.max(np.abs(got.reshape(rows, cols)[:check] - ref) / np.maximum(ref, 1e-30)) < 1e-5
    assert np.allclose(got.reshape(rows, cols).sum(-1), 1.0, atol=1e-4)


@pytest.mark.parametrize("rows,cols", [(8192, 4096), (64, 2048), (9, 576)])
def test_graph_rms_norm_is_one_row_kernel(hd, rows, cols):
    x, a = synth.normal(12, (rows, cols)), synth.uniform(13, (cols,), 0.5, 1.5)
    s, c, got = run(G.rms_norm(LB.copy(x, (rows, cols), hd), LB.copy(a, (cols,), hd), 1e-5))
    assert s.items() == ["Kernel"]
    assert c.origins() == ["warp_row_vec4" if cols <= 1024 else "row_vec4"]
    check = min(rows, 32)
    ref = oracle.gen_rms_norm(x[:check], a, 1e-5)
    assert np.max(np.abs(got.reshape(rows, cols)[:check] - ref) / np.maximum(np.abs(ref), 1e-20)) < 1e-5


def test_maps_copies_and_unaligned_shapes(hd):
    x, g = synth.normal(14, (64, 5632)), synth.normal(15, (64, 5632))
    lx, lg = LB.copy(x, x.shape, hd), LB.copy(g, g.shape, hd)
    _, c, got = run(G.silu(lx).binary(B.Mul, lg))                     # model.rs:160-168: a pure map
    assert c.origins() == ["map_vec4"]
    ref = oracle.gen_silu_mul(x, g)
    assert np.max(np.abs(got.reshape(x.shape) - ref) / np.maximum(np.abs(ref), 1e-6)) < 1e-5
    _, c, got = run(lx.binary(B.Add, lg))                              # residual add
    assert c.origins() == ["map_vec4"]
    assert np.array_equal(got.reshape(x.shape), oracle.gen_add(x, g))
    # q / k / v transposing copy (model.rs:207-215) and the GQA repeat (model.rs:80-92): pure data movement, bit exact
    q = synth.normal(16, (1, 7, 32, 64))
    _, c, got = run(LB.copy(q, q.shape, hd).transpose(2, 1))
    assert c.origins() == ["warp_row_vec4"]
    assert np.array_equal(got.reshape(1, 32, 7, 64), q.transpose(0, 2, 1, 3))
    k = synth.normal(17, (1, 4, 37, 64))
    _, c, got = run(G.repeat(LB.copy(k, k.shape, hd), 1, 8))
    assert c.origins() == ["warp_row_vec4"]
    assert np.array_equal(got.reshape(1, 32, 37, 64), np.repeat(k, 8, axis=1))
    # a row length that is not a multiple of 4 has no 128-bit form: the same kernel with one element per access
    for shape, origin in (((5, 777), "row_scalar"), ((6, 9), "warp_row_scalar")):
        y = synth.normal(18, shape)
        _, c, got = run(G.softmax(LB.copy(y, y.shape, hd)))
        assert c.origins() == [origin]
        ref = oracle.custom_softmax(y)
        assert np.max(np.abs(got.reshape(y.shape) - ref) / np.maximum(ref, 1e-30)) < 1e-5
    # the head merge of model.rs:243: transpose(2, 1) then merge_dims -- the column index splits into (head, dim)
    a = synth.normal(20, (1, 4, 8, 64))
    _, c, got = run(LB.copy(a, a.shape, hd).transpose(2, 1).merge_dims(-2))
    assert c.origins() == ["warp_row_vec4"]
    assert np.array_equal(got.reshape(1, 8, 256), a.transpose(0, 2, 1, 3).reshape(1, 8, 256))
    # a reduction over a leading dim is none of the generated shapes: per-instruction code from the SSA
    z = synth.normal(22, (8, 64))
    _, c, got = run(LB.copy(z, z.shape, hd).reduce(0, 0))
    assert c.origins() == ["ssa"]


def test_index_select_ssa_runs_on_the_gather_operator(hd):
    emb = synth.normal(19, (50, 64))
    ids = np.array([[3, 49, 0, 7, 7]], np.int32)
    y = G.index_select(LB.copy(emb, emb.shape, hd), LB.copy(ids, ids.shape, hd))
    s = Schedule.create_one(y)
    c = s.compile()
    assert s.items() == ["Ssa"] and c.origins() == ["index_select"]
    c.run()
    assert np.array_equal(y.data_vec().reshape(1, 5, 64), emb[ids[0]][None])


def test_no_item_of_an_unmodified_llama_step_is_left_on_per_instruction_code(hd):
    """Every fused kernel of ug-llama's decode step (ug-llama/src/model.rs:203-269: 14 generated kernels
    per layer) is a row, map or copy kernel of the generator; logits agree with the CPU oracle."""
    from oracle import llama_ref as R
    from ug_b200.llama import Config
    cfg = Config(hidden_size=256, intermediate_size=512, max_position_embeddings=64, num_attention_heads=4,
                 num_key_value_heads=2, num_hidden_layers=2, vocab_size=96)
    w = synth.llama_weights_f32(synth.llama_weights(cfg))
    ref = R.Model(R.Config(**cfg.__dict__), w, custom_softmax_op=False)
    model = G.Model(cfg, w, hd, custom_softmax_op=False)
    toks = synth.tokens(6, (1, 9), cfg.vocab_size)
    cache, rcache = model.new_cache(), ref.new_cache()
    seen = set()
    for lo, hi in ((0, 8), (8, 9)):
        t = LB.copy(toks[:, lo:hi], (1, hi - lo), hd)
        pos = LB.copy(np.array([[lo]], np.int32), (1, 1), hd)
        out = model.fwd(t, pos, cache)
        c = Schedule.create_one(out).compile()
        seen |= set(c.origins())
        c.run()
        got = out.data_vec().reshape(1, hi - lo, cfg.vocab_size)
        want = ref.fwd(toks[:, lo:hi], lo, rcache)
        assert np.max(np.abs(got - want)) < 1e-4 * np.abs(want).max()
    assert "ssa" not in seen, seen
    assert {"matmul", "custom", "index_select"} <= seen and seen & {"row_vec4", "warp_row_vec4"} and "map_vec4" in seen


def test_generic_kernel_takes_its_grid_per_launch(hd):
    """A one-dimensional map over [3, T] runs on ceil(3 T / 256) blocks, which is not affine in T (1 block up to
    T = 85, 2 from 86 on).  The grid is not part of what a later sighting has to match: the function generalised
    from T = 84 and 85 serves 86 and 87 with their own grids and no further compilation."""
    from ug_b200.lazy import CompilationCache
    cache, misses = CompilationCache(), []
    for t in (84, 85, 86, 87, 200):
        x = synth.normal(40 + t, (3, t))
        lx = LB.copy(x, (3, t), hd)
        y = lx.binary(B.Mul, lx).binary(B.Add, lx)
        before = cache.misses
        Schedule.create_one(y).compile(cache).run()
        misses.append(cache.misses - before)
        assert np.allclose(y.data_vec().reshape(3, t), x * x + x, rtol=1e-6, atol=1e-7)
    assert misses == [1, 1, 0, 0, 0] and cache.poly_hits == 3


def test_decode_loop_stops_compiling_once_the_kv_dependent_kernels_are_generic(hd):
    """ug-llama's step loop (ug-llama/src/main.rs:127-169: build the graph, compile_with_cache, run) over 32 tokens.
    The reference's cache keys on shapes (ug-core/src/cache.rs:8-12), so the kernels whose shape follows the KV
    length miss on every token.  Here each of them is compiled as it is on the first sighting, as a function of
    the size on the second, and never again: no miss from the third decode step on, same logits as with
    per-shape kernels, and both agree with the CPU oracle."""
    from oracle import llama_ref as R
    from ug_b200.lazy import CompilationCache
    from ug_b200.llama import Config
    cfg = Config(hidden_size=256, intermediate_size=512, max_position_embeddings=64, num_attention_heads=4,
                 num_key_value_heads=2, num_hidden_layers=2, vocab_size=96)
    w = synth.llama_weights_f32(synth.llama_weights(cfg))
    ref = R.Model(R.Config(**cfg.__dict__), w, custom_softmax_op=False)
    toks = synth.tokens(21, (1, 40), cfg.vocab_size)

    def loop(polymorphic, n_steps):
        model = G.Model(cfg, w, hd, custom_softmax_op=False)
        cache, kv = CompilationCache(), model.new_cache()
        cache.set_polymorphic(polymorphic)
        misses, logits = [], []
        # a prompt of 8 positions, then one token per step
        spans = [(0, 8)] + [(8 + i, 9 + i) for i in range(n_steps)]
        for lo, hi in spans:
            t = LB.copy(toks[:, lo:hi], (1, hi - lo), hd)
            pos = LB.copy(np.array([[lo]], np.int32), (1, 1), hd)
            out = model.fwd(t, pos, kv)
            before = cache.misses
            Schedule.create_one(out).compile(cache).run()
            misses.append(cache.misses - before)
            logits.append(out.data_vec().reshape(hi - lo, cfg.vocab_size)[-1])
        return misses, logits, cache

    misses, logits, cache = loop(True, 32)
    assert misses[1] > 0 and misses[2] > 0           # first decode step: as it is; second: the generic functions
    assert misses[3:] == [0] * 30, misses
    assert cache.poly_hits > 0
    ref_misses, ref_logits, _ = loop(False, 8)
    assert all(m > 0 for m in ref_misses[1:])        # per-shape kernels: every token compiles
    for a, b in zip(logits[:9], ref_logits):
        assert np.max(np.abs(a - b)) < 1e-5 * np.abs(b).max()
    rcache, worst = ref.new_cache(), 0.0
    for (lo, hi), got in zip([(0, 8)] + [(8 + i, 9 + i) for i in range(32)], logits):
        want = ref.fwd(toks[:, lo:hi], lo, rcache)[0, -1]
        worst = max(worst, float(np.max(np.abs(got - want)) / np.abs(want).max()))
    assert worst < 1e-4
