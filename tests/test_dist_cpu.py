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


def test_tp_shard_partitions_cover_the_model():
    """Column-parallel q/k/v/gate/up + row-parallel o/down over the shards reproduce the full products."""
    import numpy as np
    from ug_b200.dist import tp_shard
    nh, nkv, ffn, vocab, hd, hidden = 8, 2, 96, 64, 4, 32
    rng = np.random.default_rng(0)
    x = rng.standard_normal((3, hidden)).astype(np.float64)
    wq = rng.standard_normal((nh * hd, hidden))
    wo = rng.standard_normal((hidden, nh * hd))
    wg = rng.standard_normal((ffn, hidden))
    wd = rng.standard_normal((hidden, ffn))
    for size in (1, 2, 4, 8):
        shards = [tp_shard(nh, nkv, ffn, vocab, r, size) for r in range(size)]
        assert sorted(h for s in shards for h in range(s["q0"], s["q0"] + s["nq"])) == list(range(nh))
        assert sorted(f for s in shards for f in range(s["f0"], s["f0"] + s["nf"])) == list(range(ffn))
        assert sorted(v for s in shards for v in range(s["v0"], s["v0"] + s["nv"])) == list(range(vocab))
        for s in shards:   # the KV head a query head reads is one the rank holds
            for h in range(s["q0"], s["q0"] + s["nq"]):
                assert s["kv0"] <= h // (nh // nkv) < s["kv0"] + s["nkv"]
        att = sum((x @ wq[s["q0"] * hd:(s["q0"] + s["nq"]) * hd].T) @ wo[:, s["q0"] * hd:(s["q0"] + s["nq"]) * hd].T
                  for s in shards)
        assert np.allclose(att, (x @ wq.T) @ wo.T)
        mlp = sum((x @ wg[s["f0"]:s["f0"] + s["nf"]].T) @ wd[:, s["f0"]:s["f0"] + s["nf"]].T for s in shards)
        assert np.allclose(mlp, (x @ wg.T) @ wd.T)
    import pytest
    with pytest.raises(ValueError):
        tp_shard(8, 3, 96, 64, 0, 2)
