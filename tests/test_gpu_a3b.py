"""Parity at the benchmark's shapes: a 4-layer prefix (3 gated DeltaNet + 1 gated GQA, 512 experts
top-10 + shared, vocab 151936, the UD-Q4_K_XL-style type mix) of the 80B-A3B-shaped model. The
checkpoint is generated and quantised on the device; its bytes are read back for the oracle, so both
sides see identical quantised bytes.

Passes of 16 rows and more multiply some weight matrices rounded to fp16 (the tensor-core kernels, the
reference's prefill arithmetic); the oracle is told which (`Graph.fp16_weight_mask`) and rounds the same
ones, so every pass is held to the same bounds: routed sets exact except at a near-tie below 1e-3,
hidden states and logits within 1e-2."""
import numpy as np
import pytest

import modelgen
from parity import NEAR_TIE, assert_close, follow_pass, logit_gap, noise_flips, routing_flips

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def a3b4(pkg, orc):
    config = modelgen.config
    cfg = config.variant(config.A3B, n_layer=4, name="80b-a3b-shaped-4-layer-prefix")
    model = pkg.Model.synthetic(cfg, seed=0)
    tensors = {name: (typ, dims, model.read_tensor(name)) for name, typ, dims, _ in config.manifest(cfg)}
    om = orc.Model(config.graph_fields(cfg), tensors)
    return dict(model=model, oracle=om, cfg=cfg, tensors=tensors)


def test_device_generated_checkpoint_dequantises_like_the_oracle(pkg, orc, a3b4):
    for name in ("blk.0.attn_qkv.weight", "blk.3.attn_v.weight", "blk.1.ffn_gate_inp.weight"):
        typ, dims, data = a3b4["tensors"][name]
        n = 4 * dims[0]
        rb = pkg.gguf.row_bytes(typ, dims[0])
        got = pkg.dequantize(typ, data[:4 * rb], n)
        want = orc.dequantize(typ, data[:4 * rb], n)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), name
        assert 0.005 < np.std(want) < 0.04     # N(0, 0.02) survived the quantiser


def test_full_shape_prefill_and_greedy_decode_match_oracle(pkg, orc, a3b4):
    cfg = a3b4["cfg"]
    ids = np.random.default_rng(1).integers(0, cfg["vocab"], 24).astype(np.int32)
    g = pkg.Graph(a3b4["model"], n_kv=64, max_tokens=32, trace=True, use_cuda_graph=False)
    seq = a3b4["oracle"].seq()
    g.reset()
    logits, want, flips = follow_pass(g, orc, seq, ids, "24-row prefill")
    for step in range(8):
        tg, to = int(np.argmax(logits)), int(np.argmax(want))
        assert tg == to or logit_gap(want) < NEAR_TIE, (step, tg, to, logit_gap(want))
        logits, want, f2 = follow_pass(g, orc, seq, [to], f"decode step {step}")
        flips += f2
    assert len(noise_flips(flips)) <= 2, flips


def test_eighty_row_pass_routes_like_the_oracle(pkg, orc, a3b4):
    """A pass of 64 to 255 rows takes its router logits from the column-tiled mma kernel (fp16-rounded
    router weights, like the longer passes): the oracle rounds the same matrices and must route alike."""
    cfg = a3b4["cfg"]
    T = 80
    ids = np.random.default_rng(21).integers(0, cfg["vocab"], T).astype(np.int32)
    g = pkg.Graph(a3b4["model"], n_kv=96, max_tokens=128, trace=True, use_cuda_graph=False)
    assert g.fp16_weight_mask(T, 1) & pkg.lib.W16_ROUTER
    g.reset()
    follow_pass(g, orc, a3b4["oracle"].seq(), ids, "80-row pass")


def test_slots_with_long_contexts_batched_against_the_oracle(pkg, orc, a3b4):
    """Config 3's shape on the 4-layer prefix: many slots decode together, some holding a few hundred REAL
    prefilled cells, with 256-cell attention splits so that the bulk-copy-fed attention kernel of the
    64-slot benchmark runs (two splits, a ragged second one). A 16-row pass (one 16-warp DeltaNet CTA per head
    and sequence, dense projections on the tensor cores) and a 64-row pass (router logits on the mma kernel,
    work-list entries of four columns) are compared slot by slot with the oracle. Every routing decision of
    every pass, prefill included, is judged, and the oracle follows the passes' routing, so every slot stays
    comparable to the end."""
    cfg = a3b4["cfg"]
    S = 64
    rng = np.random.default_rng(33)
    lens = [int(rng.integers(2, 7)) for _ in range(S)]
    lens[0], lens[5], lens[11] = 300, 262, 391           # cells already in the cache when the batched passes run
    g = pkg.Graph(a3b4["model"], n_kv=448, max_tokens=64, slots=S, attn_split_cells=256, trace=True, use_cuda_graph=False)
    seqs, flips = [], []
    for s in range(S):
        p = rng.integers(0, cfg["vocab"], lens[s]).astype(np.int32)
        g.use_slot(s); g.reset()
        sq = a3b4["oracle"].seq()
        for o in range(0, len(p), 8):                    # passes of at most 8 rows: exact weights on both sides
            flips += follow_pass(g, orc, sq, p[o:o + 8], f"prefill of slot {s}, rows {o}..")[2]
        seqs.append(sq)
    toks = rng.integers(0, cfg["vocab"], S).astype(np.int32)
    for rows in (16, 64):
        mode = orc.DEVICE_LIKE | g.fp16_weight_mask(rows, rows)
        got = g.decode_rows(list(range(rows)), toks[:rows])
        assert g.pass_experts() > 10
        tr = g.trace(rows)
        for s in range(rows):
            forced = np.ascontiguousarray(tr["topk"][:, s:s + 1].transpose(1, 0, 2))
            want, od = seqs[s].extend([int(toks[s])], numerics=mode, trace=("hidden", "topk", "margin"), force_topk=forced)
            flips += routing_flips(tr["topk"][:, s:s + 1], od["topk"], od["margin"], f"{rows}-row pass, slot {s}")
            toks[s] = int(np.argmax(want))
            assert_close(tr["hidden"][-1][s], od["hidden"][0, -1], f"{rows}-row pass, slot {s} ({lens[s]} cells): last residual")
            assert_close(got[s], want, f"{rows}-row pass, slot {s} ({lens[s]} cells)")
            assert int(np.argmax(got[s])) == int(np.argmax(want)) or logit_gap(want) < NEAR_TIE
    decisions = (sum(lens) + 80) * cfg["n_layer"]
    assert len(noise_flips(flips)) <= decisions // 100, f"{len(noise_flips(flips))} of {decisions} routing decisions flipped above the near-tie margin: {noise_flips(flips)}"


def test_eight_slots_batched_are_each_slot_bit_for_bit(pkg, a3b4):
    """Passes of up to 8 rows run every row on the single-row schedule (routing inside the expert kernel, routing
    weights applied inside the down projection, partial rows added by the next projection): a batched step and a
    verify pass give each row exactly the logits of that row stepped alone (llm/graph_batch_test.go:36 asserts bit
    equality the same way)."""
    cfg = a3b4["cfg"]
    g = pkg.Graph(a3b4["model"], n_kv=48, max_tokens=32, slots=8, speculative=True, spec_rows=5, use_cuda_graph=False)
    rng = np.random.default_rng(19)
    toks = rng.integers(0, cfg["vocab"], 8).astype(np.int32)
    solo = []
    for s in range(8):
        g.use_slot(s); g.reset(); g.extend(rng.integers(0, cfg["vocab"], 3 + s % 4).astype(np.int32))
        ck = g.checkpoint()
        lg, _ = g.extend([int(toks[s])]); solo.append(lg)
        g.restore(ck); g.checkpoint_free(ck)
    batched = g.decode_rows(list(range(8)), toks)
    for s in range(8):
        assert np.array_equal(batched[s].view(np.uint32), solo[s].view(np.uint32)), f"slot {s}"
    # a verify pass of 5 rows against the same 5 tokens stepped one by one
    g.use_slot(0)
    rows = rng.integers(0, cfg["vocab"], 5).astype(np.int32)
    ck = g.checkpoint()
    one_by_one = [g.extend([int(t)])[0] for t in rows]
    g.restore(ck); g.checkpoint_free(ck)
    g.speculate(True)
    all_logits, _ = g.extend_rows(rows)
    g.keep(5); g.speculate(False)
    for i in range(5):
        assert np.array_equal(all_logits[i].view(np.uint32), one_by_one[i].view(np.uint32)), f"verify row {i}"


def test_sixteen_slots_batched_match_solo(pkg, a3b4):
    cfg = a3b4["cfg"]
    g = pkg.Graph(a3b4["model"], n_kv=48, max_tokens=32, slots=16, use_cuda_graph=False)
    rng = np.random.default_rng(9)
    toks = rng.integers(0, cfg["vocab"], 16).astype(np.int32)
    solo = []
    for s in range(16):
        g.use_slot(s); g.reset(); g.extend(rng.integers(0, cfg["vocab"], 3 + s % 5).astype(np.int32))
        ck = g.checkpoint()
        lg, _ = g.extend([int(toks[s])]); solo.append(lg)
        g.restore(ck); g.checkpoint_free(ck)
    batched = g.decode_rows(list(range(16)), toks)
    for s in range(16):
        # passes of 16 rows run their dense projections on fp16-rounded weights, a single row on exact ones
        assert_close(batched[s], solo[s], f"slot {s}", tol=2e-3)
        assert int(np.argmax(batched[s])) == int(np.argmax(solo[s])) or logit_gap(solo[s]) < NEAR_TIE
    # the residual row of slot r after a batched pass is row r (llm/graph.go:1454)
    assert np.isfinite(g.residual_row(15)).all()
    with pytest.raises(pkg.lib.B200Error):
        g.residual_row(16)
    first = [int(np.argmax(b)) for b in batched]
    # second step: the states and conv histories that the 16-row pass left are read by single-row passes
    # (a different DeltaNet kernel) and by another 16-row pass alike
    solo2 = []
    for s in range(16):
        g.use_slot(s)
        ck = g.checkpoint()
        lg, _ = g.extend([first[s]]); solo2.append(lg)
        g.restore(ck); g.checkpoint_free(ck)
    batched2 = g.decode_rows(list(range(16)), np.asarray(first, np.int32))
    for s in range(16):
        assert_close(batched2[s], solo2[s], f"second step, slot {s}", tol=2e-3)
    out = g.generate_greedy(list(range(16)), first, 3)
    assert out.shape == (3, 16)
    st = g.stats()
    assert st["passes"] > 30 and st["launches"] > 0 and st["device_ms"] > 0


@pytest.fixture(scope="module")
def a3b2(pkg, orc):
    config = modelgen.config
    cfg = config.variant(config.A3B, n_layer=2, full_attention_interval=2, name="80b-a3b-shaped-2-layer-prefix")
    model = pkg.Model.synthetic(cfg, seed=3)
    tensors = {name: (typ, dims, model.read_tensor(name)) for name, typ, dims, _ in config.manifest(cfg)}
    return dict(model=model, oracle=orc.Model(config.graph_fields(cfg), tensors), cfg=cfg)


def test_grouped_expert_gemm_at_512_experts_against_the_oracle(pkg, orc, a3b2):
    """One pass of 1664 rows: 32.5 rows per expert on average, so the routed experts run as the grouped
    tcgen05 GEMM over expert-sorted rows at the benchmark's 512 experts x FFN 512 (the kernel the 2048-row
    prefill of the benchmark runs). One DeltaNet and one attention layer; against the oracle with the same
    weights rounded to fp16."""
    cfg = a3b2["cfg"]
    T = 1664
    ids = np.random.default_rng(41).integers(0, cfg["vocab"], T).astype(np.int32)
    g = pkg.Graph(a3b2["model"], n_kv=T + 16, max_tokens=2048, trace=True, use_cuda_graph=False)
    mask = g.fp16_weight_mask(T, 1)
    assert mask & pkg.lib.W16_EXPERTS and mask & pkg.lib.W16_SHARED and mask & pkg.lib.W16_ROUTER
    g.reset()
    follow_pass(g, orc, a3b2["oracle"].seq(), ids, "1664-row pass")
