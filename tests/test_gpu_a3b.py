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
from parity import NEAR_TIE, NOISE_TIE, assert_close, compare, logit_gap, noise_flips, routing_flips

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


def check_pass(g, orc, seq, ids, what, min_clean=1):
    """One pass of len(ids) rows on a traced graph against the oracle in the same arithmetic."""
    T = len(ids)
    cfg = g.model.cfg
    logits, _ = g.extend(ids)
    tr = g.trace(T)
    want, ot = seq.extend(ids, numerics=orc.DEVICE_LIKE | g.fp16_weight_mask(T, 1), trace=("hidden", "topk", "margin"))
    clean, flips = routing_flips(tr["topk"], ot["topk"], ot["margin"], what)
    for l in range(cfg["n_layer"]):
        if clean[l] > 0:
            assert_close(tr["hidden"][l][:clean[l]], ot["hidden"][:clean[l], l], f"{what}: layer {l} residual, {clean[l]} of {T} rows")
        if clean[l] < T:
            # Rows after a documented near-tie: the flipped row itself differs by an expert, and later rows see it
            # through the sequence state, which can tip further boundaries. No element-wise claim there, but the
            # rows must still be the same computation: most of them route alike, and the error stays small in rms.
            rest = slice(int(clean[l]), T)
            same = np.mean([set(tr["topk"][l, t].tolist()) == set(ot["topk"][t, l].tolist()) for t in range(int(clean[l]), T)])
            r = compare(tr["hidden"][l][rest], ot["hidden"][rest, l])
            assert same >= 0.9 and r["rms"] <= 5e-2 * r["ref_rms"], f"{what}: layer {l} after the first near-tie: {same:.3f} of the rows route alike, {r}"
    assert clean[-1] >= min_clean, f"{what}: routing flips {flips} leave only {clean[-1]} comparable rows"
    assert len(noise_flips(flips)) <= 1, f"{what}: flips above the near-tie margin {noise_flips(flips)}"
    if clean[-1] == T:
        assert_close(logits, want, f"{what}: logits of the last row")
    return logits, want, flips


def test_full_shape_prefill_and_greedy_decode_match_oracle(pkg, orc, a3b4):
    cfg = a3b4["cfg"]
    ids = np.random.default_rng(1).integers(0, cfg["vocab"], 24).astype(np.int32)
    g = pkg.Graph(a3b4["model"], n_kv=64, max_tokens=32, trace=True, use_cuda_graph=False)
    seq = a3b4["oracle"].seq()
    g.reset()
    logits, want, flips = check_pass(g, orc, seq, ids, "24-row prefill", min_clean=4)
    tainted = bool(flips)
    for step in range(8):
        if not tainted:
            assert_close(logits, want, f"logits at step {step}")
            tg, to = int(np.argmax(logits)), int(np.argmax(want))
            assert tg == to or logit_gap(want) < NEAR_TIE, (step, tg, to, logit_gap(want))
        to = int(np.argmax(want))
        logits, _ = g.extend([to])
        tr = g.trace(1)
        want, od = seq.extend([to], trace=("topk", "margin"))
        _, f2 = routing_flips(tr["topk"], od["topk"], od["margin"], f"decode step {step}")
        tainted = tainted or bool(f2)


def test_eighty_row_pass_routes_like_the_oracle(pkg, orc, a3b4):
    """A pass of 64 to 255 rows takes its router logits from the column-tiled mma kernel (fp16-rounded
    router weights, like the longer passes): the oracle rounds the same matrices and must route alike."""
    cfg = a3b4["cfg"]
    T = 80
    ids = np.random.default_rng(21).integers(0, cfg["vocab"], T).astype(np.int32)
    g = pkg.Graph(a3b4["model"], n_kv=96, max_tokens=128, trace=True, use_cuda_graph=False)
    assert g.fp16_weight_mask(T, 1) & pkg.lib.W16_ROUTER
    g.reset()
    check_pass(g, orc, a3b4["oracle"].seq(), ids, "80-row pass", min_clean=8)


def prefill_both(g, orc, seq, ids, chunk, what):
    """Feeds the same tokens to a slot of the traced graph (in passes of `chunk` rows) and to the oracle and compares
    the routed sets of every row and layer. Returns True when a routing decision differed at a documented near-tie
    (the sequence state then legitimately differs from the oracle's); a difference at a clear margin fails."""
    flipped, noisy = False, []
    for o in range(0, len(ids), chunk):
        part = ids[o:o + chunk]
        g.extend(part)
        tr = g.trace(len(part))
        _, ot = seq.extend(part, numerics=orc.DEVICE_LIKE | g.fp16_weight_mask(len(part), 1), trace=("topk", "margin"), want_last=False)
        if flipped:
            continue          # the sequence states differ from here on: later decisions are no longer comparable
        _, flips = routing_flips(tr["topk"], ot["topk"], ot["margin"], f"{what}, rows {o}..{o + len(part)}")
        flipped = flipped or bool(flips)
        noisy += noise_flips(flips)
    assert len(noisy) <= max(1, len(ids) * g.model.cfg["n_layer"] // 100), f"{what}: too many flips above the near-tie margin: {noisy}"
    return flipped


def test_slots_with_long_contexts_batched_against_the_oracle(pkg, orc, a3b4):
    """Config 3's shape on the 4-layer prefix: many slots decode together, some holding a few hundred REAL
    prefilled cells, with 256-cell attention splits so that the bulk-copy-fed attention kernel of the
    64-slot benchmark runs (two splits, a ragged second one). A 16-row pass (one 16-warp DeltaNet CTA per head
    and sequence, dense projections on the tensor cores) and a 64-row pass (router logits on the mma kernel,
    work-list entries of four columns) are compared slot by slot with the oracle. Every routing decision of
    every pass, prefill included, is compared: a slot drops out of the comparison only after a documented
    near-tie flipped one of its decisions."""
    cfg = a3b4["cfg"]
    S = 64
    rng = np.random.default_rng(33)
    lens = [int(rng.integers(2, 7)) for _ in range(S)]
    lens[0], lens[5], lens[11] = 300, 262, 391           # cells already in the cache when the batched passes run
    g = pkg.Graph(a3b4["model"], n_kv=448, max_tokens=64, slots=S, attn_split_cells=256, trace=True, use_cuda_graph=False)
    seqs, near_tie = [], set()
    for s in range(S):
        p = rng.integers(0, cfg["vocab"], lens[s]).astype(np.int32)
        g.use_slot(s); g.reset()
        sq = a3b4["oracle"].seq()
        if prefill_both(g, orc, sq, p, 8, f"prefill of slot {s}"):   # passes of at most 8 rows: exact weights on both sides
            near_tie.add(s)
        seqs.append(sq)
    toks = rng.integers(0, cfg["vocab"], S).astype(np.int32)
    noisy = 0
    for rows in (16, 64):
        mode = orc.DEVICE_LIKE | g.fp16_weight_mask(rows, rows)
        got = g.decode_rows(list(range(rows)), toks[:rows])
        assert g.pass_experts() > 10
        tr = g.trace(rows)
        compared = 0
        for s in range(rows):
            want, od = seqs[s].extend([int(toks[s])], numerics=mode, trace=("topk", "margin"))
            toks[s] = int(np.argmax(want))
            if s in near_tie:
                continue
            for l in range(cfg["n_layer"]):
                if set(tr["topk"][l, s].tolist()) != set(od["topk"][0, l].tolist()):
                    # routed sets are the oracle's except at a documented near-tie
                    assert od["margin"][0, l] < NOISE_TIE, f"{rows}-row pass, slot {s}, layer {l}: routing differs at a clear margin {od['margin'][0, l]:.3e}"
                    near_tie.add(s); noisy += od["margin"][0, l] >= NEAR_TIE
                    break     # later layers see a different residual row: no longer comparable
            if s in near_tie:
                continue
            assert_close(got[s], want, f"{rows}-row pass, slot {s} ({lens[s]} cells)")
            assert int(np.argmax(got[s])) == int(np.argmax(want)) or logit_gap(want) < NEAR_TIE
            compared += 1
        assert compared >= rows * 3 // 4, (compared, sorted(near_tie))
    assert not {0, 5, 11} <= near_tie, "every long-context slot dropped out"
    assert noisy <= 3, f"{noisy} of {80 * cfg['n_layer']} batched routing decisions flipped above the near-tie margin"


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
    check_pass(g, orc, a3b2["oracle"].seq(), ids, "1664-row pass", min_clean=16)
