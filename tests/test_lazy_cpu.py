"""The host layer (lazy graph, scheduler, lowering, cache) on the CPU oracle
device: ug-core's CPU backend restated behind the same C++ Device interface.
Runs without a GPU.  Fixtures: ug-core/src/common_tests.rs and
ug-core/tests/lb_tests.rs; the emitted-C oracle forms are cross-checked
against what the restated lowering + CPU code generator produce."""
import ctypes as C

import numpy as np
import pytest

import lazy_cases as cases
import oracle
from conftest import rel_err
from oracle import llama_ref as R
from ug_b200 import synth
from ug_b200.lazy import LB, Schedule
from ug_b200.llama import Config


@pytest.fixture(scope="module")
def cpu():
    return oracle.cpu_host_device()


def _cpu_custom(cpu):
    def arr(raw, n):
        p = cpu._cpu_lib.oracle_cpu_slice_ptr(raw)
        return np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_float)), shape=(n,))

    def add_one(s):
        arr(s[1], 6)[:] = arr(s[0], 6) + 1.0

    def add_one_ip(s):
        arr(s[0], 6)[:] += 1.0
    return add_one, add_one_ip


@pytest.mark.parametrize("case", ["add", "mm", "cat", "schedule_one_kernel", "lb_copy", "schedule_broadcast",
                                  "lb_layout", "lb_set", "errors", "cache_hits"])
def test_reference_fixtures(cpu, case):
    getattr(cases, case)(cpu)


def test_custom_ops(cpu):
    cases.custom_ops(cpu, *_cpu_custom(cpu))


def test_layout_chain(cpu):
    cases.layout_chain(cpu, synth.normal(1, (2, 5, 16)))


def test_graph_softmax_pins_the_emitted_c_oracle(cpu):
    # the 2x4 known-answer vector of ug-core/tests/basic_tests.rs:41-61 through graph -> schedule -> C -> gcc
    x = np.array([[0., 1., 2., 3.], [2., 1., 2., 1.]], np.float32)
    gold = np.array([0.032058604, 0.08714432, 0.23688284, 0.6439143, 0.3655293, 0.13447072, 0.3655293, 0.13447072], np.float32)
    assert rel_err(cases.graph_softmax(cpu, x).ravel(), gold) < 3e-7
    # and the hand-written emitted-C form computes what the restated lowering + code generator emit
    x = synth.normal(2, (6, 300), 2.0)
    assert rel_err(cases.graph_softmax(cpu, x), oracle.gen_softmax(x)) < 1e-6
    lb = LB.copy(x, x.shape, cpu)
    from ug_b200 import llama_graph as G
    assert Schedule.create_one(G.softmax(lb)).items() == ["Kernel", "Kernel"]     # exp is materialised (schedule.rs:429-435)


def test_graph_rms_silu_is_one_kernel_and_matches_the_oracle(cpu):
    x, g = synth.normal(3, (5, 200)), synth.normal(4, (5, 200))
    w = synth.uniform(5, (200,), 0.5, 1.5)
    got, items = cases.graph_rms_silu(cpu, x, w, g)
    assert items == ["Kernel"]
    assert rel_err(got, oracle.gen_rms_norm_silu_gate(x, w, g, 1e-5), 1e-20) < 1e-6


def test_llama_graph_matches_llama_oracle(cpu):
    """ug-llama's Model::fwd built on the lazy graph (prefill of 5 tokens with causal mask, then two
    single-token steps) against oracle/llama_ref.py, both on the CPU."""
    from ug_b200 import llama_graph as G
    cfg = Config(hidden_size=64, intermediate_size=96, max_position_embeddings=32, num_attention_heads=4,
                 num_key_value_heads=2, num_hidden_layers=2, vocab_size=50)
    w = synth.llama_weights_f32(synth.llama_weights(cfg))
    ref = R.Model(R.Config(**cfg.__dict__), w, custom_softmax_op=False)
    toks = synth.tokens(6, (1, 7), cfg.vocab_size)
    for custom in (False, True):
        model = G.Model(cfg, w, cpu, custom_softmax_op=custom)
        cache, rcache = model.new_cache(), ref.new_cache()
        for lo, hi in ((0, 5), (5, 6), (6, 7)):
            t = LB.copy(toks[:, lo:hi], (1, hi - lo), cpu)
            pos = LB.copy(np.array([[lo]], np.int32), (1, 1), cpu)
            got = model.fwd(t, pos, cache).data_vec().reshape(1, hi - lo, cfg.vocab_size)
            want = ref.fwd(toks[:, lo:hi], lo, rcache)
            assert np.max(np.abs(got - want)) < 2e-5 * np.abs(want).max()
