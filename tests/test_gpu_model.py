"""GPU parity of the whole token loop on the tiny hybrid MoE checkpoint against the CPU oracle,
and the reference's graph invariants (chunk split, batched == solo, checkpoint, speculation),
all through the C ABI."""
import numpy as np
import pytest

import modelgen
from parity import NEAR_TIE, assert_close, compare, logit_gap

pytestmark = pytest.mark.gpu

N_PROMPT, N_GEN = 128, 128


@pytest.fixture(scope="module")
def tiny(pkg, tiny_path):
    model = pkg.Model.open(tiny_path)
    om, cfg, reader = modelgen.oracle_model(tiny_path)
    return dict(model=model, oracle=om, cfg=cfg, reader=reader)


def prompt(cfg, n, seed=1):
    return np.random.default_rng(seed).integers(0, cfg["vocab"], n).astype(np.int32)


def test_cxx_gguf_reader_agrees_with_python_reader(pkg, tiny):
    for name in ("token_embd.weight", "blk.0.attn_qkv.weight", "blk.3.attn_v.weight", "blk.1.ffn_gate_inp.weight", "blk.2.ssm_a"):
        assert np.array_equal(tiny["model"].read_tensor(name), tiny["reader"].tensors[name][2]), name
    assert tiny["model"].cfg == {k: tiny["cfg"][k] for k in tiny["model"].cfg} or \
        all(abs(tiny["model"].cfg[k] - tiny["cfg"][k]) < 1e-6 * max(1, abs(tiny["cfg"][k])) for k in tiny["model"].cfg)


def test_split_checkpoint_opens_from_any_shard(pkg, tiny, tmp_path):
    # gguf/gguf.go:748-818 OpenSet: any member names the set; an incomplete or inconsistent set is refused
    import shutil
    r = tiny["reader"]
    meta = modelgen.config.metadata(tiny["cfg"] | {"full_attention_interval": 4, "types": {}})
    paths = pkg.gguf.write_split(str(tmp_path / "tiny"), "qwen3next", meta, r.tensors, 3)
    m = pkg.Model.open(paths[1])
    for name in ("token_embd.weight", "blk.0.attn_qkv.weight", "blk.3.attn_v.weight", "output.weight"):
        assert np.array_equal(m.read_tensor(name), r.tensors[name][2]), name
    g = pkg.Graph(m, n_kv=32, use_cuda_graph=False)
    whole = pkg.Graph(tiny["model"], n_kv=32, use_cuda_graph=False)
    ids = prompt(tiny["cfg"], 5, seed=15)
    assert np.array_equal(g.forward(ids)[0].view(np.uint32), whole.forward(ids)[0].view(np.uint32))
    # a shard is missing
    d2 = tmp_path / "partial"; d2.mkdir()
    for p in paths[:2]:
        shutil.copy(p, d2)
    with pytest.raises(pkg.lib.B200Error, match="shard 3 of 3 is missing"):
        pkg.Model.open(str(d2 / "tiny-00001-of-00003.gguf"))
    # shards in the wrong places
    d3 = tmp_path / "swapped"; d3.mkdir()
    shutil.copy(paths[0], d3 / "tiny-00002-of-00003.gguf"); shutil.copy(paths[1], d3 / "tiny-00001-of-00003.gguf"); shutil.copy(paths[2], d3)
    with pytest.raises(pkg.lib.B200Error, match="split.no"):
        pkg.Model.open(str(d3 / "tiny-00001-of-00003.gguf"))


def test_prefill_matches_oracle_layer_by_layer(pkg, tiny):
    cfg = tiny["cfg"]
    ids = prompt(cfg, 24)
    g = pkg.Graph(tiny["model"], n_kv=256, max_tokens=32, trace=True, use_cuda_graph=False)
    logits, hidden = g.forward(ids)
    tr = g.trace(len(ids))
    seq = tiny["oracle"].seq()
    want_logits, ot = seq.extend(ids, trace=("hidden", "ffn_out", "topk", "topk_w", "margin"))
    for l in range(cfg["n_layer"]):
        assert_close(tr["after_mixer"][l], ot["hidden"][:, l] - ot["ffn_out"][:, l], f"layer {l} after the token mixer")
        assert_close(tr["hidden"][l], ot["hidden"][:, l], f"layer {l} residual")
        for t in range(len(ids)):
            if ot["margin"][t, l] < NEAR_TIE:
                continue   # documented near-tie: the top-k boundary is closer than 1e-3
            # the routed set is exact; the order inside it may differ where two probabilities tie
            assert set(tr["topk"][l, t].tolist()) == set(ot["topk"][t, l].tolist()), (l, t, tr["topk"][l, t], ot["topk"][t, l])
            wg = dict(zip(tr["topk"][l, t].tolist(), tr["topk_w"][l, t, :-1].tolist()))
            wo = dict(zip(ot["topk"][t, l].tolist(), ot["topk_w"][t, l].tolist()))
            assert_close([wg[e] for e in sorted(wg)], [wo[e] for e in sorted(wo)], f"routing weights {l},{t}")
    assert_close(logits, want_logits, "logits")
    assert_close(hidden, ot["hidden"][-1, -1], "last residual")


def test_greedy_decode_matches_oracle(pkg, tiny):
    """Config 1's workload: 128 prompt tokens, then 128 greedy tokens at batch 1."""
    cfg = tiny["cfg"]
    ids = prompt(cfg, N_PROMPT)
    g = pkg.Graph(tiny["model"], n_kv=N_PROMPT + N_GEN + 8, max_tokens=64)
    seq = tiny["oracle"].seq()
    logits, _ = g.forward(ids)
    want, _ = seq.extend(ids)
    near_ties = 0
    for step in range(N_GEN):
        assert_close(logits, want, f"logits at step {step}")
        tok_g, tok_o = int(np.argmax(logits)), int(np.argmax(want))
        if tok_g != tok_o:
            assert logit_gap(want) < NEAR_TIE, f"step {step}: greedy id {tok_g} != {tok_o} with gap {logit_gap(want)}"
            near_ties += 1
        tok = tok_o          # teacher forcing from the oracle after a documented near-tie
        logits, _ = g.extend([tok])
        want, _ = seq.extend([tok])
    assert near_ties <= 2


def test_exact_f32_oracle_is_within_tolerance_too(pkg, tiny):
    cfg = tiny["cfg"]
    ids = prompt(cfg, 16, seed=5)
    g = pkg.Graph(tiny["model"], n_kv=64)
    logits, _ = g.forward(ids)
    want, _ = tiny["oracle"].seq().extend(ids, numerics=0)
    r = compare(logits, want)
    assert r["max_abs"] <= 1e-2 * r["ref_max"], r


def test_chunk_split_is_the_whole_prompt(pkg, tiny):
    # llm/graph_cache_test.go TestGraphIsAChunkSplit: chunks of 16/9/2/3/1 == whole prompt
    cfg = tiny["cfg"]
    ids = prompt(cfg, 31, seed=2)
    g = pkg.Graph(tiny["model"], n_kv=64, max_tokens=32, use_cuda_graph=False)
    whole, _ = g.forward(ids)
    g.reset()
    o = 0
    for n in (16, 9, 2, 3, 1):
        part, _ = g.extend(ids[o:o + n]); o += n
    # passes of at most 8 rows normalise while staging, larger ones in a row kernel, and passes of 16 rows
    # and more run on the tensor cores with every dequantised weight rounded to fp16 (the reference's
    # prefill arithmetic): the schedules agree to a tolerance that covers that rounding
    assert_close(part, whole, "chunked prefill", tol=5e-3)
    assert int(np.argmax(part)) == int(np.argmax(whole))
    # and a chunk larger than max_tokens is cut by the library itself
    g2 = pkg.Graph(tiny["model"], n_kv=64, max_tokens=8, use_cuda_graph=False)
    cut, _ = g2.forward(ids)
    assert_close(cut, whole, "library-cut prefill", tol=5e-3)


def test_long_pass_on_the_tensor_cores_is_the_few_row_schedule(pkg, tiny):
    # 300 rows in one pass: dense projections and the experts (37 rows per expert on average) run as
    # tcgen05 GEMMs over fp16-rounded weights, the DeltaNet layers as pre-pass + scan + norm. The same
    # prompt in passes of 8 rows takes the exact-weight kernels. The two agree to the weight rounding; a
    # router near-tie that flips between them moves single rows more, so the bound on the worst element is
    # wider than the one on the whole vector.
    cfg = tiny["cfg"]
    ids = prompt(cfg, 300, seed=11)
    big = pkg.Graph(tiny["model"], n_kv=320, max_tokens=512, use_cuda_graph=False)
    small = pkg.Graph(tiny["model"], n_kv=320, max_tokens=8, use_cuda_graph=False)
    got, _ = big.forward(ids)
    want, _ = small.forward(ids)
    r = compare(got, want)
    assert r["rms"] <= 1e-2 * float(np.sqrt(np.mean(np.square(want)))), r
    assert r["max_abs"] <= 5e-2 * r["ref_max"], r
    # decoding continues from the state the long pass left
    tok = int(np.argmax(want))
    a, _ = big.extend([tok])
    b, _ = small.extend([tok])
    r = compare(a, b)
    assert r["max_abs"] <= 5e-2 * r["ref_max"], r


def test_long_attention_splits_are_the_short_ones(pkg, tiny):
    """Splits of 256 cells and more run on the bulk-copy-fed attention kernel: same logits as 64-cell splits
    and as the oracle, for ragged ends and for decode steps. Between split lengths the running maximum that the
    fp16 probabilities are rounded against differs, so the two schedules agree to 1e-3 of the largest logit."""
    cfg = tiny["cfg"]
    ids = prompt(cfg, 333, seed=11)
    seq = tiny["oracle"].seq()
    want, _ = seq.extend(ids)
    outs = []
    for split in (64, 256, 512):
        g = pkg.Graph(tiny["model"], n_kv=400, max_tokens=64, attn_split_cells=split, use_cuda_graph=False)
        logits, _ = g.forward(ids)
        assert_close(logits, want, f"prefill logits at split {split}")
        steps = [logits]
        for tok in (5, 17, 4093):
            steps.append(g.extend([tok])[0])
        outs.append(steps)
    for tok in (5, 17, 4093):
        want, _ = seq.extend([tok])
    assert_close(outs[1][-1], want, "decode logits at split 256")
    for other in outs[1:]:
        for a, b in zip(outs[0], other):
            assert_close(b, a, "long splits against short ones", tol=1e-3)


def test_tiled_prefill_attention_with_ragged_tiles_and_a_context(pkg, tiny):
    """Passes of 16 rows and more of one sequence run the tiled causal attention kernel (query tiles x key
    tiles, no split partials): a ragged last query tile, a pass that continues 50 cells of context, and key
    tiles whose last cells lie past the rows' positions, against the oracle and against the split-KV kernel
    (passes of 8 rows)."""
    cfg = tiny["cfg"]
    ids = prompt(cfg, 50 + 45 + 17, seed=19)
    seq = tiny["oracle"].seq()
    g = pkg.Graph(tiny["model"], n_kv=160, max_tokens=64, use_cuda_graph=False)
    small = pkg.Graph(tiny["model"], n_kv=160, max_tokens=8, use_cuda_graph=False)
    g.reset(); small.reset()
    o = 0
    for n in (50, 45, 17):
        got, _ = g.extend(ids[o:o + n])
        ref, _ = small.extend(ids[o:o + n])
        want, _ = seq.extend(ids[o:o + n])
        assert_close(got, want, f"pass of {n} rows after {o} cells")
        assert_close(got, ref, f"tiled against split-KV attention, {n} rows after {o} cells", tol=2e-3)
        o += n
    tok = int(np.argmax(want))
    a, _ = g.extend([tok]); b, _ = seq.extend([tok])
    assert_close(a, b, "decode after tiled prefill passes")


def test_work_list_entry_width_boundaries(pkg, tiny):
    """Passes of 32 to 128 rows build expert work-list entries of four columns, the others of eight: passes on
    both sides of each boundary (129 | 128 | 33 and 32 | 31 rows) give the oracle's logits."""
    cfg = tiny["cfg"]
    ids = prompt(cfg, 129 + 128 + 33, seed=13)
    want, _ = tiny["oracle"].seq().extend(ids)
    outs = []
    for max_tokens in (129, 128, 32, 31):
        g = pkg.Graph(tiny["model"], n_kv=320, max_tokens=max_tokens, use_cuda_graph=False)
        if max_tokens == 129:
            g.extend(ids[:129]); g.extend(ids[129:257]); logits, _ = g.extend(ids[257:])
        else:
            logits, _ = g.forward(ids)
        assert_close(logits, want, f"passes of at most {max_tokens} rows")
        outs.append(logits)
    for o in outs[1:]:
        assert_close(o, outs[0], "pass lengths against each other", tol=5e-3)


def test_decode_rows_is_each_slot(pkg, tiny):
    # llm/graph_batch_test.go TestGraphDecodeRowsIsEachSlot: batched == solo, BIT for bit: a pass of up to 8 rows
    # routes, computes and combines every row on the single-row schedule, and every projection's column depends
    # on that column alone.
    cfg = tiny["cfg"]
    g = pkg.Graph(tiny["model"], n_kv=64, max_tokens=16, slots=4, use_cuda_graph=False)
    prompts = [prompt(cfg, n, seed=10 + n) for n in (5, 9, 3)]
    toks = [7, 11, 13]
    solo = []
    for s, p in enumerate(prompts):
        g.use_slot(s); g.reset(); g.extend(p)
        ck = g.checkpoint()
        lg, _ = g.extend([toks[s]])
        solo.append(lg)
        g.restore(ck)              # back to the end of the prompt
    batched = g.decode_rows([0, 1, 2], toks)
    for s in range(3):
        assert np.array_equal(batched[s].view(np.uint32), solo[s].view(np.uint32)), f"slot {s}"
    # refusals before anything is launched (llm/batch.go:45-63)
    with pytest.raises(pkg.lib.B200Error):
        g.decode_rows([0, 0], [1, 2])
    with pytest.raises(pkg.lib.B200Error):
        g.decode_rows([9], [1])
    with pytest.raises(pkg.lib.B200Error):
        g.decode_rows([1], [cfg["vocab"]])


def test_checkpoint_is_the_prefill(pkg, tiny):
    # llm/graph_checkpoint_test.go: restoring a checkpoint and extending == never having left
    cfg = tiny["cfg"]
    ids = prompt(cfg, 20, seed=3)
    g = pkg.Graph(tiny["model"], n_kv=64, use_cuda_graph=False)
    g.forward(ids[:12])
    ck = g.checkpoint()
    a, _ = g.extend(ids[12:])
    g.restore(ck)
    assert g.past() == 12
    b, _ = g.extend(ids[12:])
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))


def test_speculative_keep_is_the_sequence(pkg, tiny):
    # llm/spec_rewind_test.go: a verify pass of n rows, keep k, equals extending by those k rows
    cfg = tiny["cfg"]
    ids = prompt(cfg, 12, seed=4)
    rows = prompt(cfg, 4, seed=6)
    g = pkg.Graph(tiny["model"], n_kv=64, speculative=True, spec_rows=4, use_cuda_graph=False)
    for k in (0, 1, 2, 4):
        g.forward(ids)
        g.speculate(True)
        all_logits, _ = g.extend_rows(rows)
        g.keep(k)
        g.speculate(False)
        assert g.past() == len(ids) + k
        nxt, _ = g.extend([5])
        plain = pkg.Graph(tiny["model"], n_kv=64, use_cuda_graph=False)
        plain.forward(ids)
        for i in range(k):
            lg, _ = plain.extend([rows[i]])
            assert np.array_equal(all_logits[i].view(np.uint32), lg.view(np.uint32)), f"verify row {i}"   # a verify row is the plain step
        want, _ = plain.extend([5])
        assert np.array_equal(nxt.view(np.uint32), want.view(np.uint32)), f"after keep({k})"


def test_device_greedy_loop_and_cuda_graph_replay(pkg, tiny):
    # the replayed step is the recorded step (llm/prerecord_test.go:48), and the device-resident
    # loop emits the ids the host loop picks
    cfg = tiny["cfg"]
    ids = prompt(cfg, 16, seed=8)
    eager = pkg.Graph(tiny["model"], n_kv=96, use_cuda_graph=False)
    replay = pkg.Graph(tiny["model"], n_kv=96, use_cuda_graph=True)
    le, _ = eager.forward(ids)
    lr, _ = replay.forward(ids)
    host_ids = []
    for _ in range(24):
        assert np.array_equal(le.view(np.uint32), lr.view(np.uint32))
        t = int(np.argmax(le)); host_ids.append(t)
        le, _ = eager.extend([t])
        lr, _ = replay.extend([t])
    dev = pkg.Graph(tiny["model"], n_kv=96, use_cuda_graph=True)
    l0, _ = dev.forward(ids)
    out = dev.generate_greedy([0], [int(np.argmax(l0))], 23)
    assert [int(np.argmax(l0))] + out[:, 0].tolist()[:-1] == host_ids[:23] or out[:, 0].tolist() == host_ids[1:24]
    assert dev.past() == len(ids) + 23
    assert dev.last_launches() > 0 and dev.last_device_ms() > 0


def test_a_wait_that_runs_out_is_reported_and_the_graph_survives(pkg, tiny):
    """Failure detection without a fault: a kernel whose bounded wait nothing can satisfy gives up, sets the
    graph's error word and returns; the pass after it reports ETIMEOUT, and the graph then works again."""
    cfg = tiny["cfg"]
    ids = prompt(cfg, 10, seed=12)
    g = pkg.Graph(tiny["model"], n_kv=64, use_cuda_graph=False)
    want, _ = g.forward(ids)
    g.inject_wait_timeout()
    with pytest.raises(pkg.lib.B200Error) as e:
        g.forward(ids)
    assert e.value.status == pkg.lib.ETIMEOUT
    again, _ = g.forward(ids)               # the error word was cleared with the report
    assert np.array_equal(again.view(np.uint32), want.view(np.uint32))


def test_extend_input_and_pass_experts(pkg, tiny):
    cfg = tiny["cfg"]
    ids = prompt(cfg, 6, seed=14)
    g = pkg.Graph(tiny["model"], n_kv=32, use_cuda_graph=False)
    a, _ = g.forward(ids)
    g.reset()
    b, hb = g.extend_input(ids)             # ExtendInput with no images is Extend (llm/graph.go:1709-1716)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
    with pytest.raises(pkg.lib.B200Error):
        g.extend_input(ids, n_images=1)     # no vision tower
    assert cfg["n_expert_used"] <= g.pass_experts() <= min(cfg["n_expert"], cfg["n_expert_used"] * len(ids))
    assert np.array_equal(g.residual_row(len(ids) - 1), hb)


def test_capacity_and_id_refusals(pkg, tiny):
    g = pkg.Graph(tiny["model"], n_kv=16)
    with pytest.raises(pkg.lib.B200Error):
        g.forward(np.zeros(17, dtype=np.int32))
    with pytest.raises(pkg.lib.B200Error):
        g.forward([-1])
    with pytest.raises(pkg.lib.B200Error):
        g.use_slot(3)
    with pytest.raises(pkg.lib.B200Error):
        g.keep(1)
