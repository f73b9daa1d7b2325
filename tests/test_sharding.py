"""Host logic of the multi-GPU row: shard plans, scatter/gather, and a world-size-2 gloo run in which each rank
processes its shard (a stand-in per-sequence function; the kernels need a GPU) and rank 0 reassembles the batch."""
import json
import os
import subprocess
import sys
import textwrap

import numpy as np

from tnn_b200 import sharding

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_contiguous_covers_and_balances():
    for batch, world in [(1024, 8), (1024, 1), (10, 4), (3, 8), (0, 2)]:
        sh = sharding.contiguous_shards(batch, world)
        assert len(sh) == world
        assert np.array_equal(np.concatenate(sh) if batch else np.zeros(0, np.int64), np.arange(batch))
        sizes = [len(s) for s in sh]
        assert max(sizes) - min(sizes) <= 1


def test_balanced_beats_contiguous_on_sorted_lengths():
    rng = np.random.default_rng(0)
    lengths = np.sort(rng.integers(16, 257, size=32))          # worst case for a contiguous split
    world = 4
    bal = sharding.balanced_shards(lengths, world, 768)
    con = sharding.contiguous_shards(len(lengths), world)
    assert sorted(np.concatenate(bal).tolist()) == list(range(32))
    assert all(len(s) == 8 for s in bal)
    lb = sharding.shard_loads(bal, lengths, 768)
    lc = sharding.shard_loads(con, lengths, 768)
    assert max(lb) < max(lc)
    assert max(lb) / (sum(lb) / world) < 1.05                   # within 5 % of a perfect split


def test_scatter_gather_roundtrip_ragged():
    rng = np.random.default_rng(1)
    x = rng.standard_normal((13, 5, 7)).astype(np.float32)
    lengths = rng.integers(1, 6, size=13)
    sh = sharding.balanced_shards(lengths, 3, 8)
    back = sharding.gather(sharding.scatter(x, sh), sh, 13)
    assert np.array_equal(back, x)


WORKER = textwrap.dedent("""
    import json, sys
    sys.path.insert(0, %r)
    import numpy as np, torch, torch.distributed as dist
    from tnn_b200 import sharding
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    rng = np.random.default_rng(0)                       # every rank derives the same plan from the same lengths
    lengths = rng.integers(4, 33, size=10)
    x = rng.standard_normal((10, 32, 8)).astype(np.float32)
    plan = sharding.balanced_shards(lengths, world, 8)
    mine = sharding.scatter(x, plan)[rank]
    y = np.cumsum(mine, axis=1) * 2.0                    # any per-sequence function stands in for the encoder
    parts = [None] * world
    dist.all_gather_object(parts, y)                     # host-side gather of results; the data path has no collective
    if rank == 0:
        out = sharding.gather(parts, plan, 10)
        print(json.dumps({"ok": bool(np.array_equal(out, np.cumsum(x, axis=1) * 2.0)),
                          "sizes": [len(p) for p in plan]}))
    dist.destroy_process_group()
""") % ROOT


def test_two_ranks_shard_and_reassemble(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                          "--master-addr", "127.0.0.1", "--master-port", "29741", str(script)],
                         capture_output=True, text=True, env=env, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [ln for ln in out.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["ok"] and d["sizes"] == [5, 5]
