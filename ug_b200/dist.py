"""Multi-GPU plumbing for the partitioned hot path: one process per GPU.

The path shards by independent units (sequences, rows, batch entries): every
rank owns a contiguous range of units and there is no data-path collective.
`torch.distributed` is used for the rendezvous, the barriers around the timed
region and the max-over-ranks of the device-side timings only (backend
``nccl`` on GPUs, ``gloo`` in the CPU tests).  The tensor-parallel variant of
the Llama engine uses it once more, to exchange the 64-byte handles of the
ranks' exchange blocks (`Group.all_gather_bytes`); its per-step sums run inside
the engine's own kernels over peer memory.
"""
import os


def env_rank():
    """(rank, local_rank, world_size) from the torchrun environment (defaults: single process)."""
    return (int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0")),
            int(os.environ.get("WORLD_SIZE", "1")))


def shard_range(n_units, rank, world):
    """Contiguous range [lo, hi) of `n_units` units owned by `rank`: sizes differ by at most one and
    the earlier ranks take the larger shares (ragged totals, fewer units than ranks included)."""
    base, extra = divmod(n_units, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def tp_shard(n_heads, n_kv_heads, ffn, vocab, rank, size):
    """What tensor-parallel rank `rank` of `size` owns: query heads [q0, q0 + nq), KV heads
    [kv0, kv0 + nkv) (one replicated KV head when there are more ranks than KV heads), FFN columns
    [f0, f0 + nf) and logit columns [v0, v0 + nv).  Mirrors ugb_llama_create_tp."""
    if n_heads % size or ffn % size or vocab % size or (n_kv_heads % size and size % n_kv_heads):
        raise ValueError(f"{size} ranks do not divide heads {n_heads} / KV heads {n_kv_heads} / ffn {ffn} / vocab {vocab}")
    nq, nf, nv = n_heads // size, ffn // size, vocab // size
    nkv = n_kv_heads // size if n_kv_heads >= size else 1
    return {"q0": rank * nq, "nq": nq, "kv0": rank * n_kv_heads // size, "nkv": nkv,
            "f0": rank * nf, "nf": nf, "v0": rank * nv, "nv": nv}


def rank_seed(seed, rank):
    """Seed of a per-rank synthetic partition: distinct per rank, reproducible."""
    return seed + 1000 * rank


class Group:
    """Process group wrapper: barrier and max / sum over ranks of host scalars."""

    def __init__(self, backend=None, device=None):
        import torch
        import torch.distributed as dist
        self.rank, self.local_rank, self.world = env_rank()
        self.dist, self.torch, self.device = dist, torch, device
        self.active = self.world > 1
        if self.active and not dist.is_initialized():
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            backend = backend or ("nccl" if torch.cuda.is_available() else "gloo")
            kw = {}
            if backend == "nccl":
                torch.cuda.set_device(self.local_rank)
                self.device = torch.device("cuda", self.local_rank)
                kw["device_id"] = self.device
            dist.init_process_group(backend, **kw)
        self.device = self.device or "cpu"

    def barrier(self):
        if self.active:
            self.dist.barrier()
            if str(self.device).startswith("cuda"):
                self.torch.cuda.synchronize()

    def _reduce(self, values, op):
        if not self.active:
            return list(values)
        t = self.torch.tensor(list(values), dtype=self.torch.float64, device=self.device)
        self.dist.all_reduce(t, op=op)
        return t.tolist()

    def max(self, values):
        """Element-wise maximum over ranks (timings: the slowest rank defines the step)."""
        return self._reduce(values, self.dist.ReduceOp.MAX)

    def sum(self, values):
        return self._reduce(values, self.dist.ReduceOp.SUM)

    def all_gather_bytes(self, payload):
        """Every rank's `payload` (bytes of one common length), in rank order."""
        if not self.active:
            return [bytes(payload)]
        t = self.torch.tensor(list(payload), dtype=self.torch.uint8, device=self.device)
        out = [self.torch.empty_like(t) for _ in range(self.world)]
        self.dist.all_gather(out, t)
        return [bytes(o.cpu().tolist()) for o in out]

    def close(self):
        if self.active and self.dist.is_initialized():
            self.dist.barrier()
            self.dist.destroy_process_group()
