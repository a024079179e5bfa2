"""Expert parallelism without a GPU: the dispatch / combine index math (strix-halo-vulkan_b200/ep.py, the host
statement of what the device kernels do) run over two gloo ranks with real exchanges, against the
single-rank result computed in slot order. No reference counterpart exists (all experts on one device,
llm/gpu_moe.go:693-705); the gate is that sharding changes no arithmetic."""
import json
import os
import subprocess
import sys

import numpy as np

from conftest import ROOT


def toy_moe(x, topk, topk_w, gate, W, Ws):
    """Single-rank result: sum over the slots in order of w_k * (W[e_k] @ x), then gate * (Ws @ x) (llm/moe.go:347-357, 403-406)."""
    out = np.zeros((x.shape[0], W.shape[1]), dtype=np.float32)
    for n in range(x.shape[0]):
        acc = np.zeros(W.shape[1], dtype=np.float32)
        for k in range(topk.shape[1]):
            acc = acc + (W[topk[n, k]] @ x[n]) * topk_w[n, k]
        out[n] = acc + (Ws @ x[n]) * gate[n]
    return out


def test_work_list_covers_every_pair_exactly_once(pkg):
    rng = np.random.default_rng(3)
    world, rows, nE, used = 4, 5, 32, 4
    topk = np.stack([rng.choice(nE, used, replace=False) for _ in range(world * rows)])
    seen = []
    for r in range(world):
        entries, cols = pkg.ep.work_list(topk, r, world, nE, entry_cols=4)
        lo, hi = pkg.ep.expert_range(r, world, nE)
        covered = np.zeros(len(cols), dtype=int)
        for e, off, n in entries:
            assert 1 <= n <= 4
            covered[off:off + n] += 1
            for p in cols[off:off + n]:
                row, slot = divmod(int(p), used + 1)
                if e < 0:
                    assert slot == used and row // rows == r          # the shared expert runs where the row lives
                else:
                    assert lo <= e < hi and topk[row, slot] == e
        assert (covered == 1).all()
        seen += cols.tolist()
    assert sorted(seen) == list(range(world * rows * (used + 1)))   # every (row, slot) pair, shared included, once
    for p in seen:
        owner, local = pkg.ep.pair_destination(p, rows, used)
        assert owner == (p // (used + 1)) // rows and 0 <= local < rows * (used + 1)


WORKER = r'''
import importlib, json, sys
sys.path.insert(0, sys.argv[1]); sys.path.insert(0, sys.argv[1] + "/tests")
import numpy as np, torch, torch.distributed as dist
from test_ep_plan import toy_moe
pkg = importlib.import_module("strix-halo-vulkan_b200")
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
rows, H, nE, used, N = 6, 32, 16, 3, 24
rng = np.random.default_rng(11)                       # the same draws on every rank
W = rng.standard_normal((nE, N, H)).astype(np.float32); Ws = rng.standard_normal((N, H)).astype(np.float32)
x_all = rng.standard_normal((world * rows, H)).astype(np.float32)
topk_all = np.stack([rng.choice(nE, used, replace=False) for _ in range(world * rows)])
w_all = rng.random((world * rows, used)).astype(np.float32); gate_all = rng.random(world * rows).astype(np.float32)
mine = slice(rank * rows, (rank + 1) * rows)
# dispatch: every rank publishes its rows and routing to all (the device stores them into every peer's buffers)
xg = [torch.empty(rows, H) for _ in range(world)]; dist.all_gather(xg, torch.from_numpy(x_all[mine].copy()))
tg = [torch.empty(rows, used, dtype=torch.int64) for _ in range(world)]; dist.all_gather(tg, torch.from_numpy(topk_all[mine].astype(np.int64)))
xg, tg = torch.cat(xg).numpy(), torch.cat(tg).numpy()
entries, cols = pkg.ep.work_list(tg, rank, world, nE, entry_cols=4)
# experts: this rank's pairs; every output row goes to the rank that owns the pair's row
send = [np.zeros((rows * (used + 1), N), dtype=np.float32) for _ in range(world)]
for e, off, n in entries:
    for p in cols[off:off + n]:
        row = int(p) // (used + 1)
        owner, local = pkg.ep.pair_destination(int(p), rows, used)
        send[owner][local] = (Ws if e < 0 else W[e]) @ xg[row]
# combine: an all-to-all of the (sparse) output buffers, as pairwise sends (gloo has no all_to_all); a pair is written
# by exactly one rank, so adding the buffers is exact
recv = [torch.empty(rows * (used + 1), N) for _ in range(world)]
reqs = [dist.isend(torch.from_numpy(send[q]), q) for q in range(world) if q != rank]
for q in range(world):
    if q != rank: dist.recv(recv[q], q)
recv[rank] = torch.from_numpy(send[rank])
for r_ in reqs: r_.wait()
down = sum(r_.numpy() for r_ in recv).reshape(rows, used + 1, N)
out = np.zeros((rows, N), dtype=np.float32)
for n in range(rows):
    acc = np.zeros(N, dtype=np.float32)
    for k in range(used):
        acc = acc + down[n, k] * w_all[mine][n, k]
    out[n] = acc + down[n, used] * gate_all[mine][n]
want = toy_moe(x_all, topk_all, w_all, gate_all, W, Ws)[mine]
res = [None] * world
dist.all_gather_object(res, bool(np.array_equal(out, want)))
if rank == 0: print(json.dumps({"equal": res}))
dist.barrier(); dist.destroy_process_group()
'''


def test_two_gloo_ranks_dispatch_and_combine_like_one_rank(tmp_path):
    w = tmp_path / "worker.py"
    w.write_text(WORKER)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29617")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
                          "--master-port", "29617", str(w), ROOT], capture_output=True, text=True, env=env, timeout=300)
    assert out.returncode == 0, out.stderr[-3000:]
    line = [l for l in out.stdout.splitlines() if l.startswith("{")][-1]
    assert json.loads(line)["equal"] == [True, True]      # bit for bit: same products, same slot order
