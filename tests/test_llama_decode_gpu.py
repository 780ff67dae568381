"""GPU parity of the fused Llama decode step against the CPU oracle of
ug-llama's forward pass (oracle/llama_ref.py), through the C ABI.

Tolerance: logits within 2e-2 of the oracle relative to the row's largest
|logit| (the stated bound for bf16 GEMM outputs and logits).  The oracle runs
f32 on bf16-rounded weights; the GPU keeps bf16 weights, bf16 KV cache and
bf16 GEMM inputs with fp32 accumulation."""
import numpy as np
import pytest

from oracle import llama_ref as R
from ug_b200 import UgError, synth
from ug_b200.llama import Config, Model

pytestmark = pytest.mark.gpu
TOL = 2e-2


def make(cfg, dev, batch, t_max, seed=100):
    w = synth.llama_weights(cfg, seed)
    gpu = Model.new(cfg, w, dev, batch, t_max)
    ref = R.Model(R.Config(**cfg.__dict__), synth.llama_weights_f32(w))
    return gpu, ref


def logit_err(got, ref):
    return float(np.max(np.abs(got - ref)) / np.max(np.abs(ref)))


def run_teacher_forced(gpu, ref, prompts, check_seqs, check_from=0):
    """Feeds prompts [batch, t] one position per step on both sides; returns the worst logit error."""
    batch, t = prompts.shape
    caches = {b: ref.new_cache() for b in check_seqs}
    worst = 0.0
    gpu.reset(0)
    for i in range(t):
        gpu.fwd(prompts[:, i])
        if i >= check_from:
            got = gpu.logits()
        for b in check_seqs:
            want = ref.fwd(prompts[b:b + 1, i:i + 1], i, caches[b])[0, 0]
            if i >= check_from:
                worst = max(worst, logit_err(got[b], want))
    return worst, caches


TINY = dict(hidden_size=128, intermediate_size=256, max_position_embeddings=1024, num_attention_heads=2,
            num_key_value_heads=1, num_hidden_layers=2, vocab_size=512)


@pytest.mark.parametrize("over", [dict(), dict(rope_interleaved=True),
                                  dict(hidden_size=512, num_attention_heads=8, num_key_value_heads=1),
                                  dict(hidden_size=256, num_attention_heads=4, num_key_value_heads=4,
                                       intermediate_size=320)])
def test_decode_matches_oracle_small(dev, over):
    cfg = Config(**{**TINY, **over})
    gpu, ref = make(cfg, dev, 16, 64)
    prompts = synth.tokens(7, (16, 21), cfg.vocab_size)
    worst, _ = run_teacher_forced(gpu, ref, prompts, check_seqs=[0, 5, 15])
    assert worst < TOL
    gpu.close()


def test_long_context_crosses_tiles_and_slices(dev):
    """T grows to 300: many 16-key sub-tiles per warp, both KV slices, ring wrap-around."""
    cfg = Config(**TINY)
    gpu, ref = make(cfg, dev, 16, 320)
    prompts = synth.tokens(8, (16, 300), cfg.vocab_size)
    worst, _ = run_teacher_forced(gpu, ref, prompts, check_seqs=[3], check_from=0)
    assert worst < TOL
    for splits in (1, 3, 8):            # slicing the KV range differently must not change the result
        gpu.set_option("att_splits", splits)
        gpu.reset(299)
        gpu.fwd(prompts[:, 299])
        base = gpu.logits()
        gpu.set_option("att_splits", 2)
        gpu.reset(299)
        gpu.fwd(prompts[:, 299])
        # slices change the running max, hence the bf16 rounding of the probabilities: not bit-equal
        assert np.max(np.abs(gpu.logits() - base)) < 5e-3 * np.abs(base).max()
    for splits in (2, 3, 4, 8):         # slices combined inside a cluster or through scratch: the same sums, same bits
        gpu.set_option("att_splits", splits)
        both = []
        for cluster in (1, 0):
            gpu.set_option("att_cluster", cluster)
            gpu.reset(299)
            gpu.fwd(prompts[:, 299])
            both.append(gpu.logits())
        assert np.array_equal(both[0], both[1])
    gpu.set_option("att_cluster", 1)
    gpu.set_option("att_splits", 2)
    gpu.reset(299)
    gpu.fwd(prompts[:, 299])
    base = gpu.logits()
    for stages in (2, 3, 4, 6):         # the ring depth only changes when a sub-tile is requested: same bits
        gpu.set_option("att_stages", stages)
        gpu.reset(299)
        gpu.fwd(prompts[:, 299])
        assert np.array_equal(gpu.logits(), base)
    gpu.close()


def test_full_width_two_layers_greedy(dev):
    """Llama-1.1B widths (2048 / 32 q heads / 4 kv heads / ffn 5632 / vocab 32000), 2 layers."""
    cfg = Config(hidden_size=2048, intermediate_size=5632, max_position_embeddings=4096,
                 num_attention_heads=32, num_key_value_heads=4, num_hidden_layers=2, vocab_size=32000)
    gpu, ref = make(cfg, dev, 16, 64)
    prompts = synth.tokens(9, (16, 35), cfg.vocab_size)
    worst, caches = run_teacher_forced(gpu, ref, prompts, check_seqs=[0, 7], check_from=30)
    assert worst < TOL
    # greedy continuation: the engine feeds its own argmax; follow it with the oracle
    toks = gpu.next_tokens()
    assert np.array_equal(toks, gpu.logits().argmax(-1).astype(np.int32))   # ties -> lowest id
    for step in range(3):
        gpu.decode(1)
        got = gpu.logits()
        for b in (0, 7):
            want = ref.fwd(np.array([[toks[b]]], np.int32), 35 + step, caches[b])[0, 0]
            assert logit_err(got[b], want) < TOL
        toks = gpu.next_tokens()
    assert gpu.position == 38
    # KV append never disturbs older positions: bit-exact comparison of the cache prefix
    k_before = gpu.kv_cache(1, 0)[:, :, :38].copy()
    gpu.decode(2)
    dev.synchronize()
    assert np.array_equal(gpu.kv_cache(1, 0)[:, :, :38], k_before)
    # and the cached keys are the oracle's roped keys rounded to bf16, within bf16 resolution
    k_ref = caches[0][1][0][0]                                    # [kv, T, d] f32
    k_gpu = synth.bf16_bits_to_f32(k_before[0])[:, :k_ref.shape[1]]
    assert np.max(np.abs(k_gpu - k_ref)) < 2e-2 * np.abs(k_ref).max()
    gpu.close()


def test_gate_up_on_cta_pairs_or_single_ctas(dev):
    """The gate|up projection of a decode step runs its k halves on a pair of CTAs (a cluster) that exchange their
    sums through shared memory, or on one CTA per tile: two summation orders of the same products, both within
    tolerance of the oracle, at a width whose last tile is partly outside (ffn 5632: 11264 = 70 x 160 + 64) and at
    a small one."""
    for over, batch in (({"hidden_size": 2048, "intermediate_size": 5632, "num_attention_heads": 32, "num_key_value_heads": 4,
                          "num_hidden_layers": 1, "vocab_size": 512, "max_position_embeddings": 128}, 64), ({}, 5)):
        cfg = Config(**{**TINY, **over})
        gpu, ref = make(cfg, dev, batch, 32)
        prompts = synth.tokens(12, (batch, 6), cfg.vocab_size)
        logits = []
        for pair in (1, 0):
            gpu.set_option("gate_up_pair", pair)
            worst, _ = run_teacher_forced(gpu, ref, prompts, check_seqs=[0, batch - 1])
            assert worst < TOL
            logits.append(gpu.logits())
        assert np.max(np.abs(logits[0] - logits[1])) < 2e-3 * np.abs(logits[1]).max()
        gpu.close()


def test_projection_timeline_is_recorded_and_ordered(dev):
    """Option gemm_profile: CTA 0 of each decode projection stamps its own clock; the stamps of a projection are
    in program order and every k block of its main loop has one."""
    import ctypes as C
    from ug_b200._lib import lib
    cfg = Config(**TINY)
    gpu, _ = make(cfg, dev, 16, 64)
    gpu.set_option("gemm_profile", 1)
    gpu.reset(0)
    gpu.fwd(synth.tokens(10, (16,), cfg.vocab_size))
    gpu.decode(2)
    buf = np.zeros(5 * 64, np.float32)
    dev._check(lib.ugb_llama_read(gpu._h, 5, buf.ctypes.data, buf.size))
    for t in buf.reshape(5, 64):
        start, dep, last_mma, acc_seen, epi, end = t[:6]
        kb = t[8:][t[8:] != 0]
        assert dep == 0 and start <= 0 and len(kb) >= 1
        assert 0 < kb[0] <= kb[-1] <= last_mma <= acc_seen <= epi <= end
        assert np.all(np.diff(kb) >= 0)
    gpu.set_option("gemm_profile", 0)
    with pytest.raises(UgError):
        dev._check(lib.ugb_llama_read(gpu._h, 5, buf.ctypes.data, buf.size))
    gpu.close()


def test_multi_step_graph_replay_equals_single_steps(dev):
    cfg = Config(**TINY)
    gpu, _ = make(cfg, dev, 16, 64)
    first = synth.tokens(10, (16,), cfg.vocab_size)
    gpu.reset(0)
    gpu.fwd(first)
    gpu.decode(6)
    a_tok, a_log = gpu.next_tokens(), gpu.logits()
    gpu.reset(0)
    gpu.fwd(first)
    for _ in range(6):
        gpu.decode(1)
    assert np.array_equal(gpu.next_tokens(), a_tok)
    assert np.array_equal(gpu.logits(), a_log)          # deterministic: fixed-order split-K sums
    gpu.close()


def test_engine_errors(dev):
    cfg = Config(**TINY)
    m = Model(cfg, dev, 16, 32)
    with pytest.raises(UgError) as e:
        m.load_weight("model.layers.0.mlp.gate_proj.weight", np.zeros((3, 3), np.uint16))
    assert e.value.code == 3 and "unexpected shape" in e.value.msg       # model.rs:142-144
    with pytest.raises(UgError) as e:
        m.load_weight("model.layers.9.mlp.gate_proj.weight", np.zeros((256, 128), np.uint16))
    assert e.value.code == 1
    with pytest.raises(UgError) as e:
        m.load_weight("lm_head.weight", np.zeros((512, 128), np.uint16))
    assert e.value.code == 1
    m.reset(31)
    m.fwd(np.zeros(16, np.int32))
    with pytest.raises(UgError) as e:
        m.decode(1)                                                      # cache is full
    assert e.value.code == 3
    m.reset(0)
    m.fwd(np.full(16, 100000, np.int32))                                 # id outside the vocabulary
    with pytest.raises(UgError) as e:
        dev.synchronize()
    assert e.value.code == 1
    with pytest.raises(UgError):
        Model(Config(**{**TINY, "hidden_size": 96, "num_attention_heads": 2}), dev, 16, 32)   # head_dim 48
    with pytest.raises(UgError):
        Model(cfg, dev, 129, 32)                                         # more sequences than one GEMM row tile
    m.close()


@pytest.mark.parametrize("batch", [1, 5])
def test_decode_small_batches(dev, batch):
    """Fewer sequences than the 16 rows of an MMA row group: the unused rows are zero-filled tiles."""
    cfg = Config(**TINY)
    gpu, ref = make(cfg, dev, batch, 64)
    prompts = synth.tokens(17, (batch, 12), cfg.vocab_size)
    worst, _ = run_teacher_forced(gpu, ref, prompts, check_seqs=sorted({0, batch - 1}))
    assert worst < TOL
    gpu.close()


@pytest.mark.parametrize("bn", [80, 96, 128, 256])
def test_gemm_tile_widths_agree(dev, bn):
    """Every projection on another tile width (80 / 96 leave a ragged last tile and a partly used
    32-column accumulator chunk) reproduces the default configuration's logits."""
    cfg = Config(**{**TINY, "hidden_size": 256, "num_attention_heads": 4, "intermediate_size": 352})
    gpu, ref = make(cfg, dev, 16, 64)
    prompts = synth.tokens(19, (16, 9), cfg.vocab_size)
    worst, _ = run_teacher_forced(gpu, ref, prompts, check_seqs=[4])
    assert worst < TOL
    base = gpu.logits()
    for key in ("bn_qkv", "bn_o", "bn_gate_up", "bn_down", "bn_lm_head"):
        gpu.set_option(key, bn)
    gpu.set_option("gemm_smem_kib", 64)
    worst, _ = run_teacher_forced(gpu, ref, prompts, check_seqs=[4])
    assert worst < TOL
    assert np.max(np.abs(gpu.logits() - base)) < 2e-3 * np.abs(base).max()
    gpu.close()


def test_attention_front_end_variants_are_bit_identical(dev):
    """Work moved in front of griddepcontrol.wait (the attention kernel's K / V ring, the norm kernel's
    residual row) and the TMA fetch path change when bytes are requested, not what is computed: logits and
    chosen tokens are bit for bit the same.  The early paths switch themselves on only for shapes whose
    projections cannot be co-resident (the condition under which they are race-free), hence the wide model."""
    cfg = Config(hidden_size=1536, intermediate_size=4864, max_position_embeddings=256, num_attention_heads=24,
                 num_key_value_heads=4, num_hidden_layers=2, vocab_size=1024)
    gpu = Model.new(cfg, synth.llama_weights(cfg, 31), dev, 64, 128)
    prompts = synth.tokens(23, (64, 50), cfg.vocab_size)
    results = []
    for early, tma in ((1, 0), (0, 0), (1, 1), (0, 1)):
        gpu.set_option("att_early", early)
        gpu.set_option("att_tma", tma)
        gpu.reset(0)
        gpu.prefill(prompts)
        gpu.decode(30)                                # crosses sub-tile and ring boundaries
        results.append((gpu.logits(), gpu.next_tokens()))
        dev.synchronize()
    for lg, tk in results[1:]:
        assert np.array_equal(lg, results[0][0]) and np.array_equal(tk, results[0][1])
    gpu.close()
