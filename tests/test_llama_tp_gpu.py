"""Tensor-parallel variant of the Llama engine.

One GPU: the single-rank instance of the exchange kernels (rank 0 of 1) must reproduce the plain
engine bit for bit.  Two or more GPUs: tests/tp_worker.py under torchrun, one process per GPU,
checked against the CPU oracle (logits within 2e-2 of the largest |logit|)."""
import os
import subprocess
import sys

import numpy as np
import pytest

from ug_b200 import synth
from ug_b200.llama import Config, Model

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

TINY = dict(hidden_size=256, intermediate_size=512, max_position_embeddings=512, num_attention_heads=4,
            num_key_value_heads=2, num_hidden_layers=2, vocab_size=512)


def test_single_rank_exchange_path_is_bit_identical(dev):
    cfg = Config(**TINY)
    w = synth.llama_weights(cfg, 77)
    prompts = synth.tokens(5, (16, 40), cfg.vocab_size)
    plain = Model.new(cfg, w, dev, 16, 64)
    tp = Model.new(cfg, w, dev, 16, 64, tp=(0, 1))
    assert (tp.tp_rank, tp.tp_size, tp.vocab_local, tp.vocab_offset) == (0, 1, cfg.vocab_size, 0)
    for m in (plain, tp):
        m.prefill(prompts[:, :33], all_logits=True)
    assert np.array_equal(plain.prefill_logits(), tp.prefill_logits())
    for i in range(33, 40):
        for m in (plain, tp):
            m.fwd(prompts[:, i])
        assert np.array_equal(plain.logits(), tp.logits())
    for m in (plain, tp):
        m.decode(4)
    assert np.array_equal(plain.next_tokens(), tp.next_tokens())
    assert np.array_equal(plain.logits(), tp.logits())
    dev.synchronize()
    plain.close()
    tp.close()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_tensor_parallel_ranks_match_oracle(world):
    import torch
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(29600 + world), os.path.join(ROOT, "tests", "tp_worker.py")]
    out = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0 and "TP_WORKER_OK" in out.stdout, out.stdout[-3000:] + out.stderr[-3000:]
