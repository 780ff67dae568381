"""The multi-process plumbing of the partitioned path on CPU: two gloo ranks
agree on the unit ranges, take the max over ranks of their timings and sum
their unit counts, which is exactly what bench.py does around the timed
region at N > 1."""
import os
import subprocess
import sys
import textwrap

import pytest

from ug_b200 import dist as D

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("n,world", [(64, 1), (64, 2), (64, 8), (7, 4), (3, 8), (0, 2)])
def test_shard_range_partitions_every_unit_once(n, world):
    ranges = [D.shard_range(n, r, world) for r in range(world)]
    assert ranges[0][0] == 0 and ranges[-1][1] == n
    assert all(a[1] == b[0] for a, b in zip(ranges, ranges[1:]))
    sizes = [hi - lo for lo, hi in ranges]
    assert max(sizes) - min(sizes) <= 1 and sizes == sorted(sizes, reverse=True)


def test_rank_seeds_are_distinct():
    assert len({D.rank_seed(8, r) for r in range(8)}) == 8


WORKER = textwrap.dedent("""
    import sys
    sys.path.insert(0, %r)
    from ug_b200 import dist as D
    g = D.Group(backend="gloo")
    lo, hi = D.shard_range(65, g.rank, g.world)
    g.barrier()
    ms = g.max([1.5 + g.rank, 10.0 - g.rank])          # per-rank timings -> slowest rank
    units = g.sum([hi - lo])
    g.barrier()
    if g.rank == 0:
        print("RESULT", g.world, ms, units, flush=True)
    g.close()
""")


def test_two_gloo_ranks_reduce_timings_and_units(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER % ROOT)
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                          "--master-addr", "127.0.0.1", "--master-port", "29533", str(script)],
                         capture_output=True, text=True, timeout=240)
    assert out.returncode == 0, out.stderr[-2000:]
    line = [l for l in out.stdout.splitlines() if l.startswith("RESULT")]
    assert line == ["RESULT 2 [2.5, 10.0] [65.0]"]
