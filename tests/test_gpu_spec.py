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
