"""Expert parallelism on the GPU. With one rank the exchange runs against itself (same kernels, same flags,
no peer): the pass must be the plain pass bit for bit. With two GPUs, two ranks in this process (one graph
per device, a thread each) decode their own slots with the routed experts split between them and must give
the logits of one GPU that holds all slots and all experts."""
import threading

import numpy as np
import pytest

import modelgen
from parity import NEAR_TIE, assert_close, follow_pass, logit_gap, routing_flips

pytestmark = pytest.mark.gpu


def prompt(cfg, n, seed):
    return np.random.default_rng(seed).integers(0, cfg["vocab"], n).astype(np.int32)


def fill(g, cfg, slots, seed0):
    for s in range(slots):
        g.use_slot(s); g.reset(); g.extend(prompt(cfg, 4 + s % 5, seed0 + s))


@pytest.mark.parametrize("rows", [3, 8, 16])
def test_one_rank_exchanging_with_itself_is_the_plain_pass(pkg, orc, tiny_path, rows):
    model = pkg.Model.open(tiny_path)
    om, cfg, _ = modelgen.oracle_model(tiny_path)
    toks = prompt(cfg, rows, 77)
    g = pkg.Graph(model, n_kv=48, max_tokens=32, slots=rows, trace=True, use_cuda_graph=False)
    seqs = []
    for s in range(rows):
        g.use_slot(s); g.reset()
        seqs.append(om.seq())
        follow_pass(g, orc, seqs[-1], prompt(cfg, 4 + s % 5, 100 + s), f"prefill of slot {s}")
    pkg.Graph.ep_connect_local([g])
    g.ep_enable(True)
    got = g.decode_rows(list(range(rows)), toks)
    tr = g.trace(rows)
    for s in range(rows):       # against the oracle, which follows the pass's routing
        forced = np.ascontiguousarray(tr["topk"][:, s:s + 1].transpose(1, 0, 2))
        want, od = seqs[s].extend([int(toks[s])], numerics=orc.DEVICE_LIKE | g.fp16_weight_mask(rows, rows), trace=("topk", "margin"), force_topk=forced)
        routing_flips(tr["topk"][:, s:s + 1], od["topk"], od["margin"], f"slot {s}")
        assert_close(got[s], want, f"exchanged pass, slot {s}")
    if rows > 8:
        # from 9 rows the exchanged pass runs the kernels of the plain pass on the same work per pair: bit for bit
        plain = pkg.Graph(model, n_kv=48, max_tokens=32, slots=rows, use_cuda_graph=False)
        fill(plain, cfg, rows, 100)
        want = plain.decode_rows(list(range(rows)), toks)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    # the replayed (captured) step exchanges too
    g2 = pkg.Graph(model, n_kv=48, max_tokens=32, slots=rows, use_cuda_graph=True)
    fill(g2, cfg, rows, 100)
    pkg.Graph.ep_connect_local([g2]); g2.ep_enable(True)
    a = g2.decode_rows(list(range(rows)), toks)
    assert np.array_equal(a.view(np.uint32), got.view(np.uint32))
    out = g2.generate_greedy(list(range(rows)), [int(np.argmax(r)) for r in a], 3)
    assert out.shape == (3, rows)
    assert g2.stats()["expert_streams"] > 0


def test_expert_parallel_refusals(pkg, tiny_path):
    model = pkg.Model.open(tiny_path)
    g = pkg.Graph(model, n_kv=32, max_tokens=8, slots=8, use_cuda_graph=False)
    with pytest.raises(pkg.lib.B200Error):
        g.ep_enable(True)                                   # nothing attached yet
    with pytest.raises(pkg.lib.B200Error):
        g.ep_export(0, 3)                                   # 32 experts do not divide over 3 ranks
    other = pkg.Graph(model, n_kv=32, max_tokens=8, slots=8, use_cuda_graph=False)
    with pytest.raises(pkg.lib.B200Error, match="GPU of its own"):
        pkg.Graph.ep_connect_local([g, other])              # two ranks on one GPU would wait for each other


def test_two_ranks_on_two_gpus_match_one_gpu(pkg, tiny_path):
    if pkg.lib.load().b200_device_count() < 2:
        pytest.skip("needs two GPUs")
    world, rows = 2, 6
    cfg = pkg.Model.open(tiny_path).cfg
    models = [pkg.Model.open(tiny_path, device=d) for d in range(world)]
    # one GPU, all slots, all experts
    whole = pkg.Graph(models[0], n_kv=48, max_tokens=32, slots=world * rows, use_cuda_graph=False)
    fill(whole, cfg, world * rows, 300)
    toks = prompt(cfg, world * rows, 78)
    want = whole.decode_rows(list(range(world * rows)), toks)
    want2 = whole.decode_rows(list(range(world * rows)), [int(np.argmax(r)) for r in want])
    # two ranks: rank r holds slots [r * rows, (r + 1) * rows) as its local slots 0..rows-1
    graphs = []
    for r in range(world):
        g = pkg.Graph(models[r], n_kv=48, max_tokens=32, slots=rows, use_cuda_graph=True)
        for s in range(rows):
            g.use_slot(s); g.reset(); g.extend(prompt(cfg, 4 + (r * rows + s) % 5, 300 + r * rows + s))
        graphs.append(g)
    pkg.Graph.ep_connect_local(graphs)
    for g in graphs:
        g.ep_enable(True)
    got, errs = [None] * world, []

    def step(r, ids, out):
        try:
            out[r] = graphs[r].decode_rows(list(range(rows)), ids[r * rows:(r + 1) * rows])
        except Exception as e:  # surfaced below
            errs.append(e)

    for ids, ref in ((toks, want), (np.asarray([int(np.argmax(r)) for r in want], np.int32), want2)):
        th = [threading.Thread(target=step, args=(r, ids, got)) for r in range(world)]
        [t.start() for t in th]; [t.join() for t in th]
        assert not errs, errs
        for r in range(world):
            for s in range(rows):
                assert_close(got[r][s], ref[r * rows + s], f"rank {r} slot {s}", tol=1e-3)
                assert int(np.argmax(got[r][s])) == int(np.argmax(ref[r * rows + s])) or logit_gap(ref[r * rows + s]) < NEAR_TIE
