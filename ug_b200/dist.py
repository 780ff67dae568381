"""Multi-GPU plumbing for the partitioned hot path: one process per GPU.

The path shards by independent units (sequences, rows, batch entries): every
rank owns a contiguous range of units and there is no data-path collective.
`torch.distributed` is used for the rendezvous, the barriers around the timed
region and the max-over-ranks of the device-side timings only (backend
``nccl`` on GPUs, ``gloo`` in the CPU tests).
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

    def close(self):
        if self.active and self.dist.is_initialized():
            self.dist.barrier()
            self.dist.destroy_process_group()
