"""The benchmark's multi-rank plumbing on CPU: two gloo ranks agree on max-over-ranks timing and rank 0
alone reports (the N > 1 path of bench.py without a GPU)."""
import os
import subprocess
import sys

from conftest import ROOT

WORKER = r'''
import os, sys, json
sys.path.insert(0, sys.argv[1])
import torch, torch.distributed as dist
import bench
dist.init_process_group("gloo")
rank = dist.get_rank()
ms = bench.max_over_ranks(10.0 + 5.0 * rank, world=dist.get_world_size(), device="cpu")
total = bench.whole_job_rate(units_per_rank=128, world=dist.get_world_size(), ms=ms)
if rank == 0:
    print(json.dumps({"ms": ms, "rate": total}))
dist.barrier()
dist.destroy_process_group()
'''


def test_two_gloo_ranks_report_the_slowest_rank_and_the_whole_job(tmp_path):
    w = tmp_path / "worker.py"
    w.write_text(WORKER)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29611")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
                          "--master-port", "29611", str(w), ROOT], capture_output=True, text=True, env=env, timeout=240)
    assert out.returncode == 0, out.stderr[-2000:]
    import json
    line = [l for l in out.stdout.splitlines() if l.startswith("{")][-1]
    r = json.loads(line)
    assert abs(r["ms"] - 15.0) < 1e-6                 # the slower rank
    assert abs(r["rate"] - 2 * 128 / 0.015) < 1e-3    # both ranks' units over that time
