"""CPU, world size 2 over gloo: the rank plumbing bench.py uses for N > 1 (shard selection, barrier, max-over-ranks
reduction, rank-0-only reporting).  No kernel runs here."""
import os
import subprocess
import sys
import textwrap

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = textwrap.dedent("""
    import os, sys, json
    sys.path.insert(0, %r)
    import torch, torch.distributed as dist
    import bench
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    # every rank draws its own batch (seed offset by rank): shards are disjoint work, weights identical
    from tnn_b200 import model_synth
    wl = model_synth.make_workload(model_synth.BERT_BASE, 2, 16, seed=rank, num_layers=1)
    ms = torch.tensor([10.0 + rank, 20.0 - rank], dtype=torch.float64)
    agg = bench.reduce_max_over_ranks(ms, world)
    seqs = world * 2 * 5
    value = seqs / (float(agg[0]) / 1e3)
    dist.barrier()
    if rank == 0:
        print(json.dumps({"world": world, "ms": agg.tolist(), "value": value, "x0": float(wl.x[0, 0, 0])}))
    dist.destroy_process_group()
""") % ROOT


def test_two_ranks_reduce_max_and_rank0_reports(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                          "--master-addr", "127.0.0.1", "--master-port", "29731", str(script)],
                         capture_output=True, text=True, env=env, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    import json
    lines = [ln for ln in out.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1                      # only rank 0 prints
    d = json.loads(lines[0])
    assert d["world"] == 2
    assert d["ms"] == [11.0, 20.0]              # max over ranks of each timing
    assert abs(d["value"] - 20 / 0.011) < 1e-6  # all ranks' sequences over the slowest rank's time
