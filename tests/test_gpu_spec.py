"""MTP draft head and speculative decoding on the GPU: the draft layer against the oracle, and the
reference's gate that speculative output is plain greedy output (llm/spec_slots_test.go:199
TestServedSpeculationIsPlain, backend/llm_spec_test.go:36)."""
import numpy as np
import pytest

import modelgen
from parity import assert_close

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def drafted(pkg, orc):
    cfg = modelgen.config.variant(modelgen.config.TINY, name="tiny-hybrid-moe-mtp", has_draft=1)
    path = modelgen.cached_gguf(cfg)
    om, ocfg, _ = modelgen.oracle_model(path)
    return dict(model=pkg.Model.open(path), oracle=om, cfg=ocfg)


def plain_greedy(pkg, model, ids, n):
    g = pkg.Graph(model, n_kv=len(ids) + n + 8, use_cuda_graph=False)
    lg, _ = g.forward(ids)
    out = []
    for _ in range(n):
        t = int(np.argmax(lg)); out.append(t)
        lg, _ = g.extend([t])
    return out


def test_draft_rows_match_the_oracle(pkg, drafted):
    cfg = drafted["cfg"]
    assert cfg["has_draft"] == 1
    ids = np.random.default_rng(3).integers(0, cfg["vocab"], 12).astype(np.int32)
    g = pkg.Graph(drafted["model"], n_kv=64, max_tokens=16, use_cuda_graph=False)
    _, res = g.extend_residual(ids)
    seq = drafted["oracle"].seq()
    _, ot = seq.extend(ids, trace=("hidden",))
    want_res = ot["hidden"][:, -1]            # residual after the last trunk layer
    assert_close(res, want_res, "trunk residual rows")
    # prime the draft with (h_j, x_{j+1}) for the whole prompt, then one chained step
    dres, dlg = g.draft_rows(want_res[:-1], ids[1:], 0)
    ds = drafted["oracle"].draft_seq()
    for j in range(len(ids) - 1):
        h_o, lg_o = ds.draft_step(want_res[j], int(ids[j + 1]))
        assert_close(dres[j], h_o, f"draft residual row {j}")
        assert_close(dlg[j], lg_o, f"draft logits row {j}")
    tok = int(np.argmax(lg_o))
    dres2, dlg2 = g.draft_rows(h_o[None, :], [tok], 4096)
    h_o2, lg_o2 = ds.draft_step(h_o, tok, draft_vocab=4096)
    assert dlg2.shape == (1, 4096)
    assert_close(dres2[0], h_o2, "chained draft residual")
    assert_close(dlg2[0], lg_o2, "chained draft logits over the vocabulary prefix")
    assert g.draft_past() == len(ids)


@pytest.mark.parametrize("depth", [1, 2, 4])
def test_speculative_output_is_plain_greedy(pkg, drafted, depth):
    cfg = drafted["cfg"]
    ids = np.random.default_rng(5).integers(0, cfg["vocab"], 20).astype(np.int32)
    n_out = 24
    want = plain_greedy(pkg, drafted["model"], ids, n_out)
    # (a) the real draft head: random weights, so it is almost always rejected
    g = pkg.Graph(drafted["model"], n_kv=96, max_tokens=32, speculative=True, spec_rows=depth + 1, use_cuda_graph=False)
    sp = pkg.spec.Speculator(g, depth=depth)
    got = [sp.prime(ids)]
    while len(got) < n_out:
        got += sp.round()
    assert got[:n_out] == want
    # (b) a proposer that knows the future is always accepted: depth + 1 tokens a round
    g2 = pkg.Graph(drafted["model"], n_kv=96, max_tokens=32, speculative=True, spec_rows=depth + 1, use_cuda_graph=False)
    sp2 = pkg.spec.Speculator(g2, depth=depth)
    got2 = [sp2.prime(ids)]
    while len(got2) < n_out:
        base = len(got2)
        got2 += sp2.round(propose=lambda lg, k: want[base + k] if base + k < len(want) else 0)
    assert got2[:n_out] == want
    assert sp2.stats["accepted"] >= sp2.stats["rounds"] * depth - depth
    # (c) a proposer that is right for the first draft only: keeps exactly two tokens a round
    g3 = pkg.Graph(drafted["model"], n_kv=96, max_tokens=32, speculative=True, spec_rows=depth + 1, use_cuda_graph=False)
    sp3 = pkg.spec.Speculator(g3, depth=depth)
    got3 = [sp3.prime(ids)]
    while len(got3) < n_out:
        base = len(got3)
        got3 += sp3.round(propose=lambda lg, k: want[base] if (k == 0 and base < len(want)) else cfg["vocab"] - 1)
    assert got3[:n_out] == want


def test_slotted_speculation_is_plain_greedy_per_slot(pkg, drafted):
    """Config 5's batch shape on the tiny model: several sequences speculate over ONE slotted graph and one
    slotted draft cache, their rounds interleaved; every slot emits its own plain greedy sequence
    (llm/spec_slots_test.go:199 TestServedSpeculationIsPlain)."""
    cfg = drafted["cfg"]
    S, n_out, depth = 4, 12, 2
    rng = np.random.default_rng(17)
    prompts = [rng.integers(0, cfg["vocab"], 9 + 3 * s).astype(np.int32) for s in range(S)]
    want = [plain_greedy(pkg, drafted["model"], p, n_out) for p in prompts]
    g = pkg.Graph(drafted["model"], n_kv=96, max_tokens=32, slots=S, speculative=True, spec_rows=depth + 1, use_cuda_graph=False)
    assert g.draft_slots() == S and g.draft_max_rows() >= depth + 1 and g.draft_wide() == cfg["n_embd"]
    sps = [pkg.spec.Speculator(g, depth=depth, slot=s) for s in range(S)]
    got = [[sp.prime(p)] for sp, p in zip(sps, prompts)]
    rnd = 0
    while any(len(o) < n_out for o in got):
        for s in ((0, 2, 1, 3) if rnd % 2 else (3, 1, 0, 2)):     # interleave in changing orders
            if len(got[s]) < n_out:
                base = len(got[s])
                # slot 1 gets a proposer that knows the future, the others the real (random) draft head
                prop = (lambda lg, k, b=base, w=want[s]: w[b + k] if b + k < len(w) else 0) if s == 1 else None
                got[s] += sps[s].round(propose=prop)
        rnd += 1
    for s in range(S):
        assert got[s][:n_out] == want[s], s
    assert sps[1].stats["accepted"] > 0


def test_speculate_first_and_draft_vocabulary(pkg, drafted):
    cfg = drafted["cfg"]
    g = pkg.Graph(drafted["model"], n_kv=32, speculative=True, spec_rows=3, use_cuda_graph=False)
    plain = pkg.Graph(drafted["model"], n_kv=32, use_cuda_graph=False)
    g.forward([1, 2, 3]); plain.forward([1, 2, 3])
    assert not g.speculating()
    g.speculate(True); g.speculate_first(True)
    assert g.speculating()
    g.extend_rows([7, 8, 9])
    with pytest.raises(pkg.lib.B200Error):
        g.rewind()                          # with SpeculateFirst a pass ends by Commit or KeepFirst (llm/graph.go:1166)
    g.keep_first()
    assert g.past() == 4
    g.speculate(False)
    a, _ = g.extend([5]); plain.extend([7]); b, _ = plain.extend([5])
    assert_close(a, b, "after keep_first", tol=1e-3)
    # SetVocab: draft logits over the first k ids only (llm/mtp.go:675)
    with pytest.raises(pkg.lib.B200Error):
        g.draft_set_vocab(1000)             # not a multiple of 16
    g.draft_set_vocab(4096)
    _, res = plain.extend_residual([11, 12])
    _, lg = g.draft_rows(res[:1], [12])
    assert lg.shape == (1, 4096)
    g.draft_reset()
    assert g.draft_past() == 0


def test_speculation_refusals(pkg, drafted):
    g = pkg.Graph(drafted["model"], n_kv=32, speculative=True, spec_rows=3, use_cuda_graph=False)
    g.forward([1, 2, 3])
    g.speculate(True)
    with pytest.raises(pkg.lib.B200Error):
        g.extend_rows([1, 2, 3, 4])          # more rows than spec_rows
    g.extend_rows([1, 2])
    with pytest.raises(pkg.lib.B200Error):
        g.keep(3)
    g.rewind()
    assert g.past() == 3
    plain = pkg.Graph(drafted["model"], n_kv=32, use_cuda_graph=False)
    with pytest.raises(pkg.lib.B200Error):
        plain.speculate(True)
