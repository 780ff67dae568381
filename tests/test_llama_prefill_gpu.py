"""GPU parity of the causal prefill path (Model::fwd with seq_len > 1) against
the CPU oracle of ug-llama's forward pass, through the C ABI.

Tolerance: logits within 2e-2 of the oracle relative to the largest |logit| of
the sequence (the stated bound for bf16 GEMM outputs and logits); KV-cache
entries written by prefill and by one-token steps agree to one bf16 rounding
step of the largest entry (the projections run with different tile shapes,
hence different fp32 summation orders, before the rounding)."""
import numpy as np
import pytest

from oracle import llama_ref as R
from ug_b200 import UgError, synth
from ug_b200.llama import Config, Model

pytestmark = pytest.mark.gpu
TOL = 2e-2

TINY = dict(hidden_size=128, intermediate_size=256, max_position_embeddings=1024, num_attention_heads=2,
            num_key_value_heads=1, num_hidden_layers=2, vocab_size=512)


def make(cfg, dev, batch, t_max, seed=100):
    w = synth.llama_weights(cfg, seed)
    gpu = Model.new(cfg, w, dev, batch, t_max)
    ref = R.Model(R.Config(**cfg.__dict__), synth.llama_weights_f32(w))
    return gpu, ref


def logit_err(got, ref):
    return float(np.max(np.abs(got - ref)) / np.max(np.abs(ref)))


@pytest.mark.parametrize("over,batch,t", [
    (dict(), 4, 21),                                  # less than one query tile
    (dict(rope_interleaved=True), 3, 64),             # exactly one tile, odd batch
    (dict(hidden_size=512, num_attention_heads=8, num_key_value_heads=1), 2, 150),   # ragged last tile, 8 heads per KV head
    (dict(hidden_size=256, num_attention_heads=4, num_key_value_heads=4, intermediate_size=320), 8, 130),
    (dict(), 1, 1),                                   # a block of one position
])
@pytest.mark.parametrize("tc", [0, 1, 2])
def test_prefill_matches_oracle(dev, over, batch, t, tc):
    """tc = 1: attention on the tcgen05 / TMEM kernel (128-query tiles, work items drawn from a counter), 2: the
    same with the items dealt round-robin, 0: on the mma.sync kernel (64-query tiles)."""
    cfg = Config(**{**TINY, **over})
    gpu, ref = make(cfg, dev, batch, 256)
    gpu.set_option("prefill_attention_tc", tc)
    prompts = synth.tokens(7, (batch, t), cfg.vocab_size)
    gpu.prefill(prompts, all_logits=True)
    got = gpu.prefill_logits()
    assert got.shape == (batch, t, cfg.vocab_size)
    last = gpu.logits()
    for b in sorted({0, batch // 2, batch - 1}):
        want = ref.fwd(prompts[b:b + 1], 0, ref.new_cache())[0]
        assert logit_err(got[b], want) < TOL
        assert logit_err(last[b], want[-1]) < TOL
    assert gpu.position == t
    assert np.array_equal(gpu.next_tokens(), np.argmax(last, axis=1).astype(np.int32))
    gpu.close()


@pytest.mark.parametrize("tc", [0, 1])
def test_chunked_prefill_and_continuation(dev, tc):
    """Chunks of 16 positions (prefill_rows 64 at batch 4) give the logits of one whole block, and
    prefill(t1) followed by prefill(t2) continues at cache position t1."""
    cfg = Config(**TINY)
    prompts = synth.tokens(9, (4, 100), cfg.vocab_size)
    whole, ref = make(cfg, dev, 4, 128)
    whole.set_option("prefill_attention_tc", tc)
    whole.prefill(prompts, all_logits=True)
    base = whole.prefill_logits()
    want = ref.fwd(prompts[1:2], 0, ref.new_cache())[0]
    assert logit_err(base[1], want) < TOL

    chunked, _ = make(cfg, dev, 4, 128)
    chunked.set_option("prefill_attention_tc", tc)
    chunked.set_option("prefill_rows", 64)
    chunked.prefill(prompts, all_logits=True)
    got = chunked.prefill_logits()
    assert logit_err(got[1], want) < TOL
    assert np.max(np.abs(got - base)) < 5e-3 * np.abs(base).max()
    with pytest.raises(UgError):
        chunked.set_option("prefill_rows", 128)      # workspace already sized

    chunked.reset(0)
    chunked.prefill(prompts[:, :37])
    chunked.prefill(prompts[:, 37:], all_logits=True)
    tail = chunked.prefill_logits()
    assert tail.shape == (4, 63, cfg.vocab_size)
    assert np.max(np.abs(tail - base[:, 37:])) < 5e-3 * np.abs(base).max()
    assert chunked.position == 100
    whole.close()
    chunked.close()


def test_prefill_then_greedy_decode_matches_stepwise(dev):
    """The cache a prefill leaves is the cache one-token steps leave, and greedy decoding continues from it."""
    cfg = Config(**TINY)
    batch, t, n_new = 16, 70, 6
    prompts = synth.tokens(11, (batch, t), cfg.vocab_size)
    a, ref = make(cfg, dev, batch, 96)
    b, _ = make(cfg, dev, batch, 96)
    a.prefill(prompts)
    for i in range(t):
        b.fwd(prompts[:, i])
    la, lb = a.logits(), b.logits()
    assert np.max(np.abs(la - lb)) < 5e-3 * np.abs(lb).max()
    for layer in range(cfg.num_hidden_layers):
        for which in (0, 1):
            ka = synth.bf16_bits_to_f32(a.kv_cache(layer, which))[:, :, :t]
            kb = synth.bf16_bits_to_f32(b.kv_cache(layer, which))[:, :, :t]
            assert np.max(np.abs(ka - kb)) <= 2.0 ** -7 * np.abs(kb).max()
    # greedy continuation against the oracle fed with the tokens the GPU chose
    cache = ref.new_cache()
    ref.fwd(prompts[2:3], 0, cache)
    tok = a.next_tokens()
    for s in range(n_new):
        a.decode(1)
        want = ref.fwd(np.array([[tok[2]]], np.int32), t + s, cache)[0, 0]
        assert logit_err(a.logits()[2], want) < TOL
        tok = a.next_tokens()
    assert a.position == t + n_new
    a.close()
    b.close()


def test_prefill_rejects_bad_arguments(dev):
    cfg = Config(**TINY)
    gpu, _ = make(cfg, dev, 2, 64)
    with pytest.raises(UgError):
        gpu.prefill(synth.tokens(1, (2, 65), cfg.vocab_size))        # longer than the cache
    with pytest.raises(UgError):
        gpu.prefill(synth.tokens(1, (3, 8), cfg.vocab_size))         # wrong batch
    with pytest.raises(UgError):
        gpu.prefill_logits()                                          # nothing kept yet
    bad = synth.tokens(1, (2, 8), cfg.vocab_size)
    bad[1, 3] = cfg.vocab_size + 5
    gpu.prefill(bad)
    with pytest.raises(UgError):
        dev.synchronize()                                             # out-of-range id raises the status word
    gpu.close()


@pytest.mark.parametrize("tc", [1, 2])
def test_prefill_config4_shape(dev, tc):
    """Llama-1.1B widths, 8 sequences x 512 positions (2 layers to keep the oracle in seconds): 1024 attention
    work items of 2 to 8 key tiles over 296 persistent CTAs, so every CTA runs several items back to back.
    Both ways of handing out the items give the same bits, and a second pass over the same prompts repeats them
    (the work counter is back at zero after each launch)."""
    cfg = Config(hidden_size=2048, intermediate_size=5632, max_position_embeddings=2048, num_attention_heads=32,
                 num_key_value_heads=4, num_hidden_layers=2, vocab_size=32000)
    gpu, ref = make(cfg, dev, 8, 512)
    gpu.set_option("prefill_attention_tc", tc)
    prompts = synth.tokens(13, (8, 512), cfg.vocab_size)
    gpu.prefill(prompts, all_logits=True)
    got = gpu.prefill_logits()
    want = ref.fwd(prompts[5:6], 0, ref.new_cache())[0]
    assert logit_err(got[5], want) < TOL
    for other in (3 - tc, tc):
        gpu.set_option("prefill_attention_tc", other)
        gpu.reset(0)
        gpu.prefill(prompts, all_logits=True)
        assert np.array_equal(gpu.prefill_logits(), got)
    gpu.close()


@pytest.mark.parametrize("tc", [0, 1, 2])
def test_long_prefill_many_key_tiles(dev, tc):
    """1100 positions in chunks of 256 and 300: up to 18 key tiles per query tile on the tcgen05 kernel (every
    barrier's phase wraps many times), a ragged last tile, and chunks that start inside a key tile."""
    cfg = Config(**{**TINY, "max_position_embeddings": 2048})
    gpu, ref = make(cfg, dev, 2, 1152)
    gpu.set_option("prefill_attention_tc", tc)
    gpu.set_option("prefill_rows", 512)               # 256 positions per chunk at batch 2
    prompts = synth.tokens(15, (2, 1100), cfg.vocab_size)
    gpu.prefill(prompts[:, :300])                      # the second call starts at cache position 300
    gpu.prefill(prompts[:, 300:], all_logits=True)
    got = gpu.prefill_logits()
    want = ref.fwd(prompts[1:2], 0, ref.new_cache())[0]
    assert logit_err(got[1], want[300:]) < TOL
    assert gpu.position == 1100
    gpu.close()
