"""One rank of the tensor-parallel parity check (launched by torchrun from test_llama_tp_gpu.py).

Every rank builds its share of the same model, runs a chunked prefill and greedy decode steps, and
the ranks' logit slices are gathered on the host.  Rank 0 compares them with the CPU oracle of
ug-llama's forward pass and with the single-rank engine on the same GPU; every rank checks that the
ranks chose the same tokens."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    import torch
    import torch.distributed as dist
    import ug_b200
    from ug_b200 import synth
    from ug_b200.dist import Group
    from ug_b200.llama import Config, Model

    group = Group(backend="nccl")
    rank, world = group.rank, group.world
    dev = ug_b200.Device(group.local_rank)
    cases = [dict(hidden_size=512, intermediate_size=1024, max_position_embeddings=512, num_attention_heads=8,
                  num_key_value_heads=2, num_hidden_layers=3, vocab_size=1024),
             dict(hidden_size=512, intermediate_size=768, max_position_embeddings=512, num_attention_heads=8,
                  num_key_value_heads=1, num_hidden_layers=2, vocab_size=512, rope_interleaved=True)]
    batch, t, n_new = 4, 90, 5
    for ci, over in enumerate(cases):
        cfg = Config(**over)
        w = synth.llama_weights(cfg, 300 + ci)
        prompts = synth.tokens(21 + ci, (batch, t), cfg.vocab_size)
        m = Model.new(cfg, w, dev, batch, 128, tp=(rank, world), group=group)
        m.set_option("prefill_rows", 128)                 # 32 positions per chunk: three chunks
        m.prefill(prompts, all_logits=True)
        local = [m.prefill_logits()]                      # [batch, t, vocab / world]
        toks = [m.next_tokens()]
        for _ in range(n_new):
            m.decode(1)
            local.append(m.logits()[:, None, :])
            toks.append(m.next_tokens())
        dev.synchronize()
        mine = torch.from_numpy(np.ascontiguousarray(np.concatenate(local, axis=1))).cuda(group.local_rank)
        parts = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(parts, mine)
        full = np.concatenate([p.cpu().numpy() for p in parts], axis=2)          # [batch, t + n_new, vocab]
        tk = torch.from_numpy(np.stack(toks)).cuda(group.local_rank)
        tks = [torch.empty_like(tk) for _ in range(world)]
        dist.all_gather(tks, tk)
        for other in tks:
            assert torch.equal(other, tk), "ranks chose different tokens"
        assert np.array_equal(np.stack(toks)[0], np.argmax(full[:, t - 1], axis=1)), "greedy choice is not the argmax of the gathered logits"
        if rank == 0:
            from oracle import llama_ref as R
            ref = R.Model(R.Config(**cfg.__dict__), synth.llama_weights_f32(w))
            cache = ref.new_cache()
            want = ref.fwd(prompts[1:2], 0, cache)[0]
            err = float(np.max(np.abs(full[1, :t] - want)) / np.max(np.abs(want)))
            assert err < 2e-2, f"prefill logits vs oracle: {err}"
            for s in range(n_new):
                want = ref.fwd(np.array([[np.stack(toks)[s, 1]]], np.int32), t + s, cache)[0, 0]
                err = float(np.max(np.abs(full[1, t + s] - want)) / np.max(np.abs(want)))
                assert err < 2e-2, f"decode step {s} logits vs oracle: {err}"
            single = Model.new(cfg, w, dev, batch, 128)
            single.set_option("prefill_rows", 128)
            single.prefill(prompts, all_logits=True)
            base = single.prefill_logits()
            d = float(np.max(np.abs(full[:, :t] - base)) / np.max(np.abs(base)))
            assert d < 5e-3, f"tensor-parallel vs single-rank logits: {d}"
            single.close()
            print(f"case {ci}: ok (world {world})", flush=True)
        m.close()
        group.barrier()
    group.close()
    if rank == 0:
        print("TP_WORKER_OK", flush=True)


if __name__ == "__main__":
    main()
