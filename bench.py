"""Decode benchmark of the B200 token loop.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One step = one greedy decode token at batch 1 of the 80B-A3B-shaped Q4_K hybrid MoE model
(48 layers, 512 experts top-10 + shared) after a 2048-token random prompt, fp16 KV cache.
Weights are synthetic (seeded N(0, 0.02), quantised on the device by the library's own
quantiser); token ids are uniform random. `value` is the device-resident greedy loop (ids never
leave the GPU); `e2e` is the same step through the reference-facing call: one token id in from
host memory, the full logits row out to pinned host memory, argmax on the host.
"""
import argparse
import importlib
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# dram__bytes_read.sum + dram__bytes_write.sum of one decode step, from an ncu capture of the 4-layer prefix
# (`--profile 1 --layers 4` under ncu's dram byte counters) scaled to 36 DeltaNet + 12 attention layers + head. The
# figure belongs to the kernels it was captured on: profiles/decode_step_a3b_dram_traffic.md names them, and it is
# re-captured whenever the kernels of the single-row step change (set it to None until then).
A3B_DRAM_BYTES_PER_STEP = 2500.6e6
PROMPT = 2048
METRIC = "decode tok/s at batch 1 (Q4_K hybrid MoE, 80B-A3B shape)"


def measured_peak_gbs():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def algorithmic_bytes_per_token(pkg, cfg, ctx):
    """Bytes one decode step has to move: every weight row it needs once, the DeltaNet state
    read and written, the conv inputs written, and the KV cells read (+1 written)."""
    gguf, config = pkg.gguf, pkg.config
    H, nE, used, ff = cfg["n_embd"], cfg["n_expert"], cfg["n_expert_used"], cfg["ffn_expert"]
    w = 0
    for name, typ, dims, _ in config.manifest(cfg):
        if name.startswith(f"blk.{cfg['n_layer']}."):
            continue                                          # the draft layer is not part of a plain decode step
        nbytes = gguf.tensor_bytes(typ, dims)
        if name == "token_embd.weight":
            nbytes = gguf.row_bytes(typ, dims[0])            # one row is gathered
        elif "_exps." in name:
            nbytes = nbytes // nE * used                      # only the routed experts stream
        w += nbytes
    n_dn = sum(0 if config.is_attention_layer(cfg, l) else 1 for l in range(cfg["n_layer"]))
    n_at = cfg["n_layer"] - n_dn
    state = n_dn * cfg["dn_heads_v"] * cfg["dn_head_dim"] ** 2 * 4 * 2
    ring = n_dn * (2 * cfg["dn_heads_k"] + cfg["dn_heads_v"]) * cfg["dn_head_dim"] * 4
    kv = n_at * 2 * cfg["n_head_kv"] * cfg["head_dim"] * 2 * (ctx + 1)
    return w + state + ring + kv


def max_over_ranks(value, world, device="cuda"):
    """A duration as the slowest rank saw it."""
    if world <= 1:
        return float(value)
    import torch
    import torch.distributed as dist
    t = torch.tensor([float(value)], device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def whole_job_rate(units_per_rank, world, ms):
    """Units all ranks processed per second: every rank decodes its own sequences (no exchange step)."""
    return world * units_per_rank / (ms / 1e3)


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs."""

    def __init__(self, index):
        self.samples, self._stop, self.index = [], threading.Event(), index
        self._t = threading.Thread(target=self._run, daemon=True)

    def _run(self):
        q = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown," \
            "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader,nounits", "-i", str(self.index)],
                                     capture_output=True, text=True, timeout=5).stdout.strip().split(",")
                self.samples.append([s.strip() for s in out])
            except Exception:
                pass
            self._stop.wait(0.2)

    def __enter__(self):
        self._t.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        self._t.join(timeout=3)

    def summary(self):
        sm = [float(s[0]) for s in self.samples if len(s) >= 6 and s[0].replace(".", "").isdigit()]
        mx = [float(s[1]) for s in self.samples if len(s) >= 6 and s[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for s in self.samples if len(s) >= 6 for n, v in zip(names, s[2:6]) if v.lower().startswith("active")})
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(sm)}


def batched_bytes(pkg, cfg, slots, ctx, streams_per_step):
    """Algorithmic bytes of one batched step on one GPU: dense weights once, every routed expert the step actually
    streamed (counted on the device, summed over layers), every local slot's DeltaNet state read + written and
    its KV cells read."""
    gguf, config = pkg.gguf, pkg.config
    nE = cfg["n_expert"]
    dense = expert_one = 0
    for name, typ, dims, _ in config.manifest(cfg):
        if name.startswith(f"blk.{cfg['n_layer']}."):
            continue                                          # the draft layer is not part of a plain decode step
        nb = gguf.tensor_bytes(typ, dims)
        if name == "token_embd.weight":
            nb = gguf.row_bytes(typ, dims[0]) * slots
        if "_exps." in name:
            expert_one += nb // nE
        else:
            dense += nb
    n_dn = sum(0 if config.is_attention_layer(cfg, l) else 1 for l in range(cfg["n_layer"]))
    n_at = cfg["n_layer"] - n_dn
    state = n_dn * cfg["dn_heads_v"] * cfg["dn_head_dim"] ** 2 * 4 * 2 * slots
    kv = n_at * 2 * cfg["n_head_kv"] * cfg["head_dim"] * 2 * float(np.sum(ctx))
    return dense + expert_one / cfg["n_layer"] * streams_per_step + state + kv


def batched_decode(pkg, model, cfg, total_slots, steps, rank, world, dist, barrier):
    """BASELINE config 3: `total_slots` sequences in all, split evenly over the ranks (strong scaling), each with a
    seeded context of 8192..32768 cells that is declared prefilled over seeded NON-ZERO caches and DeltaNet state,
    decoding greedily together. Two arms in the same run: every rank computes the experts of its own rows
    (`slot_split`: model replicated, no exchange), and the routed experts sharded over the ranks with dispatch /
    combine exchanges over NVLink peer memory (`expert_parallel`)."""
    per = total_slots // world
    if per * world != total_slots:
        return {"error": f"{total_slots} slots do not divide over {world} ranks"}
    g = pkg.Graph(model, n_kv=32768 + 2 * steps + 48, max_tokens=max(total_slots, 8), slots=per, use_cuda_graph=True)
    all_ctx = np.random.default_rng(7).integers(8192, 32769, total_slots)      # the same 64 contexts whatever the rank count
    ctx = all_ctx[rank * per:(rank + 1) * per]
    for s in range(per):
        g.use_slot(s)
        g.synth_context(int(ctx[s]), seed=1000 + rank * per + s)
    first = np.random.default_rng(8).integers(0, cfg["vocab"], total_slots).astype(np.int32)[rank * per:(rank + 1) * per]
    ids = list(range(per))
    peak, which = measured_peak_gbs()
    out = {"slots_total": total_slots, "slots_per_gpu": per, "n_gpus": world, "unit": "tok/s", "scaling": "strong",
           "mean_context": float(np.mean(all_ctx)), "peak_source": which,
           "contexts": "seeded lengths 8192..32768 declared prefilled over seeded non-zero fp16 K/V and DeltaNet state"}
    arms = ["slot_split"] + (["expert_parallel"] if world > 1 else [])
    if world > 1:
        def gather(b):
            res = [None] * world
            dist.all_gather_object(res, b)
            return res
        pkg.ep.connect(g, rank, world, gather)
        g.ep_enable(False)
    for arm in arms:
        g.ep_enable(arm == "expert_parallel") if world > 1 else None
        for s in range(per):
            g.use_slot(s); g.set_past(int(ctx[s]))
        barrier()
        toks = g.generate_greedy(ids, first, 3)                                 # warm-up, graph capture
        g.stats_reset()
        barrier()
        toks = g.generate_greedy(ids, toks[-1], steps)
        ms = g.last_device_ms() / steps
        streams = g.stats()["expert_streams"] / steps
        nbytes = batched_bytes(pkg, cfg, per, ctx + 3 + steps / 2, streams)
        ms_all = max_over_ranks(ms, world)
        out[arm] = {"ms_per_step": ms_all, "value": total_slots / (ms_all / 1e3), "experts_streamed_per_step_rank0": streams,
                    "algorithmic_bytes_per_step_rank0": nbytes, "roofline_frac_rank0": nbytes / (ms / 1e3) / 1e9 / peak,
                    "launches_per_step": g.last_launches()}
    g.destroy()
    best = max(arms, key=lambda a: out[a]["value"])
    out["value"], out["ms_per_step"], out["best_arm"] = out[best]["value"], out[best]["ms_per_step"], best
    return out


def cpu_baseline(pkg, cfg, device, tokens=8):
    """The CPU oracle (a port of the reference's CPU code) on this host's cores, on a bounded sample: decode on a
    4-layer and a 12-layer prefix-shaped model (head included), extrapolated linearly to 48 layers. The 12-layer
    model is also the parity leg: the same quantised bytes run on the GPU and through the oracle in its device-like
    mode, greedy ids compared token by token under teacher forcing from the oracle."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import orc
    orc.build()
    config = pkg.config
    times, parity = {}, None
    for nl in (4, 12):
        sub = config.variant(cfg, n_layer=nl, has_draft=0, name=f"{cfg['name']}-{nl}-layer")
        gm = pkg.Model.synthetic(sub, seed=0, device=device)
        tensors = {name: (typ, dims, gm.read_tensor(name)) for name, typ, dims, _ in config.manifest(sub)}
        om = orc.Model(config.graph_fields(sub), tensors)
        seq = om.seq()
        ids = np.random.default_rng(1).integers(0, cfg["vocab"], 16).astype(np.int32)
        seq.extend(ids[:4], numerics=orc.EXACT)
        t = time.perf_counter()
        for i in range(tokens):
            seq.extend([int(ids[i % 4])], numerics=orc.EXACT)
        times[nl] = (time.perf_counter() - t) / tokens
        if nl == 12:
            g = pkg.Graph(gm, n_kv=64, max_tokens=8, use_cuda_graph=True)
            pseq = om.seq()
            for o in range(0, 16, 8):                     # passes of 8 rows: exact weights on both sides
                lg, _ = g.extend(ids[o:o + 8])
            want, tr = pseq.extend(ids, trace=("margin",))
            mism = ties = 0
            worst = float(np.abs(lg - want).max() / np.abs(want).max())
            n_cmp = 12
            for _ in range(n_cmp):
                tg, to = int(np.argmax(lg)), orc.argmax(want)
                gap = float(np.sort(want)[-1] - np.sort(want)[-2])
                tie = gap < 1e-3 or bool((tr["margin"] < 1e-3).any())
                ties += tie
                mism += (tg != to) and not tie
                lg, _ = g.extend([to])
                want, tr = pseq.extend([to], trace=("margin",))
                worst = max(worst, float(np.abs(lg - want).max() / np.abs(want).max()))
            parity = {"model": sub["name"], "tokens_compared": n_cmp, "id_mismatches": int(mism), "near_ties": int(ties),
                      "max_logit_err_over_scale": worst, "oracle_mode": "device-like (fp16 matmul inputs, exact weights)"}
            g.destroy()
        del seq, om, tensors
        gm.close()
    per_token = times[4] + (times[12] - times[4]) * (cfg["n_layer"] - 4) / 8.0
    cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else os.cpu_count()
    return {"value": 1.0 / per_token, "unit": "tok/s", "cores": cores, "kind": "port",
            "sample": f"exact-f32 CPU oracle, {tokens} decode tokens each on a 4- and a 12-layer model of the same shape (head included) "
                      f"at short context, extrapolated linearly to {cfg['n_layer']} layers "
                      f"({times[4] * 1e3:.0f} ms and {times[12] * 1e3:.0f} ms per token)"}, parity


def verify_pass_times(pkg, model, cfg, prompt, torch):
    """MTP speculation: time of one verify pass of 1..5 rows on the trunk through the
    speculative API (rows written to per-row state planes, then rewound). With random draft and trunk weights
    acceptance is ~1/vocab, so only the rows -> pass-time ratio is reported, never a speed-up."""
    g = pkg.Graph(model, n_kv=len(prompt) + 64, max_tokens=512, slots=1, speculative=True, spec_rows=5, use_cuda_graph=False)
    g.forward(prompt)
    ids = np.random.default_rng(5).integers(0, cfg["vocab"], 5).astype(np.int32)
    out = {}
    for rows in (1, 2, 3, 5):
        g.speculate(True)
        for it in range(3 + 12):
            if it == 3:
                torch.cuda.synchronize(); t0 = time.perf_counter()
            g.extend_rows(ids[:rows]); g.rewind()
        torch.cuda.synchronize()
        out[str(rows)] = round((time.perf_counter() - t0) / 12 * 1e3, 3)
        g.speculate(False)
    g.destroy()
    return {"verify_pass_ms_by_rows": out, "context": len(prompt),
            "note": "host-timed through extend_rows (every row's logits copied to the host); rows -> time ratio only"}


def speculative_decode(pkg, model, cfg, torch, batch, prompt_len, n_out, depths=(1, 2, 4)):
    """BASELINE config 5: MTP speculative decoding with the 1-layer draft head (gated GQA attention + 512-expert MoE,
    random Q4_K-mix weights), every round verified in one trunk pass. `batch` sequences share one slotted graph and
    draft cache, their rounds interleaved. With independent random draft and trunk weights nothing is accepted, so
    what is reported is the cost of a round against a plain greedy step, and that the emitted ids ARE the plain
    greedy ids."""
    rng = np.random.default_rng(11)
    prompts = [rng.integers(0, cfg["vocab"], prompt_len).astype(np.int32) for _ in range(batch)]
    # plain greedy ids of every sequence (the reference: llm/spec_slots_test.go:199 compares with exactly this)
    gp = pkg.Graph(model, n_kv=prompt_len + n_out + 8, max_tokens=2048, slots=batch, use_cuda_graph=True)
    firsts = []
    for s in range(batch):
        gp.use_slot(s)
        lg, _ = gp.forward(prompts[s])
        firsts.append(int(np.argmax(lg)))
    # every sequence's plain greedy ids, stepped alone (the arithmetic of a verify pass's rows)
    cks = []
    for s in range(batch):
        gp.use_slot(s); cks.append(gp.checkpoint())
    plain_ids = [[firsts[s]] + gp.generate_greedy([s], [firsts[s]], n_out - 1)[:, 0].tolist() for s in range(batch)]
    for s in range(batch):
        gp.use_slot(s); gp.restore(cks[s]); gp.checkpoint_free(cks[s])
    torch.cuda.synchronize(); t0 = time.perf_counter()
    gp.generate_greedy(list(range(batch)), firsts, n_out - 1)
    torch.cuda.synchronize()
    plain_ms = (time.perf_counter() - t0) / (n_out - 1) * 1e3        # one batched greedy step
    gp.destroy()
    out = {"batch": batch, "prompt_tokens": prompt_len, "output_tokens": n_out, "plain_batched_step_ms": round(plain_ms, 3), "depths": {}}
    for depth in depths:
        g = pkg.Graph(model, n_kv=prompt_len + n_out + 16, max_tokens=2048, slots=batch, speculative=True, spec_rows=depth + 1, use_cuda_graph=False)
        sps = [pkg.spec.Speculator(g, depth=depth, draft_vocab=65536, slot=s) for s in range(batch)]
        got = [[sp.prime(p)] for sp, p in zip(sps, prompts)]
        torch.cuda.synchronize(); t0 = time.perf_counter()
        rounds = 0
        while any(len(o) < n_out for o in got):
            for s in range(batch):
                if len(got[s]) < n_out:
                    got[s] += sps[s].round(room=n_out - len(got[s]) + 1)
                    rounds += 1
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        same = all(got[s][:n_out] == plain_ids[s][:n_out] for s in range(batch))
        acc = sum(sp.stats["accepted"] for sp in sps)
        out["depths"][str(depth)] = {"round_ms": round(dt / rounds * 1e3, 3), "tokens_per_round": round(sum(len(o) for o in got) / rounds, 3),
                                     "accepted_drafts": acc, "ids_equal_plain_greedy": bool(same)}
        g.destroy()
    out["note"] = "a round = draft steps (draft head over the first 65536 ids) + one verify pass of depth + 1 rows through the host loop " \
                  "(llm/spec.go:703-852); rounds of the batch's sequences are interleaved one slot at a time, as the reference's scheduler speculates only " \
                  "for a conversation that decodes alone (backend/llm_sched.go:940-954)"
    return out


def prefill_config4(pkg, model, cfg, torch, n=32768, chunk=4096):
    """BASELINE config 4: one n-token uniform-random prompt in passes of `chunk` rows: K-quant tcgen05 GEMMs for the
    projections and the experts, the chunked (64-token) gated delta rule, tiled causal attention writing the fp16 cache."""
    g = pkg.Graph(model, n_kv=n + 16, max_tokens=chunk, slots=1, use_cuda_graph=False)
    ids = np.random.default_rng(13).integers(0, cfg["vocab"], n).astype(np.int32)
    g.forward(ids[:chunk])                      # first-use set-up, untimed
    g.stats_reset()
    torch.cuda.synchronize(); t0 = time.perf_counter()
    g.forward(ids)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    st = g.stats()
    g.destroy()
    # algorithmic flops: 2 x active weights per token, plus attention 4 * ctx * head_dim * heads per layer, plus the delta rule
    gguf, config = pkg.gguf, pkg.config
    active = 0
    for name, typ, dims, _ in config.manifest(cfg):
        if name == "token_embd.weight" or name.startswith(f"blk.{cfg['n_layer']}."):
            continue
        k = int(np.prod(dims))
        active += k // cfg["n_expert"] * cfg["n_expert_used"] if "_exps." in name else k
    active -= cfg["vocab"] * cfg["n_embd"] * (1 - 1.0 / n)          # the head runs for the last row only
    n_at = sum(1 for l in range(cfg["n_layer"]) if config.is_attention_layer(cfg, l))
    n_dn = cfg["n_layer"] - n_at
    attn = 4.0 * (n / 2) * cfg["head_dim"] * cfg["n_head"] * n_at
    dn = 6.0 * cfg["dn_head_dim"] ** 2 * cfg["dn_heads_v"] * n_dn
    flops_tok = 2.0 * active + attn + dn
    return {"prompt_tokens": n, "chunk": chunk, "value": n / dt, "unit": "tok/s", "seconds": round(dt, 3), "passes": st["passes"],
            "device_ms": round(st["device_ms"], 1), "gflop_per_token": round(flops_tok / 1e9, 2),
            "achieved_tflops": round(flops_tok * n / dt / 1e12, 1), "launches_per_pass": st["last_launches"]}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=16)
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--config", default="a3b", help="a3b (the benchmark) or tiny (a quick functional run)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--slots", type=int, default=64, help="also time batched decode over this many slots (0 = skip)")
    ap.add_argument("--prompt", type=int, default=0, help="override the prompt length (profiling runs)")
    ap.add_argument("--chunk", type=int, default=2048, help="rows per prefill pass (the graph's max_tokens)")
    ap.add_argument("--layers", type=int, default=0, help="keep only the first N layers (small cases for profiler captures)")
    ap.add_argument("--profile-prefill", type=int, default=0, help="run one prefill pass of N rows between cudaProfilerStart/Stop and exit")
    ap.add_argument("--profile-batch", type=int, default=0, help="run N eager batched decode steps over --slots slots between cudaProfilerStart/Stop and exit")
    ap.add_argument("--profile", type=int, default=0, help="run N eager decode steps between cudaProfilerStart/Stop and exit")
    args = ap.parse_args()
    # torchrun exports OMP_NUM_THREADS=1 to its workers; the CPU legs (rank 0 only) are meant to use every core
    # the process may run on, and libgomp reads the variable when the oracle library is loaded
    ncores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    if int(os.environ.get("OMP_NUM_THREADS", "0") or 0) < ncores:
        os.environ["OMP_NUM_THREADS"] = str(ncores)
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    pkg = importlib.import_module("strix-halo-vulkan_b200")
    cfg = pkg.config.CONFIGS[args.config]
    if args.config == "a3b" and not args.layers:
        cfg = pkg.config.variant(cfg, has_draft=1)       # blk.48: the MTP draft layer (config 5); the trunk is the same 48 layers
    if args.layers:
        cfg = pkg.config.variant(cfg, n_layer=args.layers, name=f"{cfg['name']}-{args.layers}-layer-prefix")
    prompt_len = args.prompt or (PROMPT if args.config == "a3b" else 128)
    steps, warmup = args.steps, max(args.warmup, 3)

    import torch
    import torch.distributed as dist
    if args.impl == "reference" and rank != 0:
        # rank 0 alone times the CPU implementation. The other ranks leave at once, before any process group
        # exists: a rank parked in a barrier spins on a host core, and every OpenMP barrier of the timed code
        # would then wait for the thread that shares that core.
        return
    if world > 1 and args.impl != "reference":
        import datetime
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank), timeout=datetime.timedelta(seconds=300))
    torch.cuda.set_device(local_rank)

    if args.impl == "reference":
        # the reference's own CPU implementation of the path (the oracle port), rank 0 only
        if rank == 0:
            cb, parity = cpu_baseline(pkg, cfg, local_rank, tokens=max(steps, 4) if steps <= 32 else 8)
            line = {"impl": "reference", "metric": METRIC, "value": cb["value"], "unit": "tok/s", "n_gpus": args.gpus, "steps": steps,
                    "warmup": warmup, "ms_per_step": 1e3 / cb["value"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                    "dtype": "f32", "data": "synthetic",
                    "config": {"workload": "batch-1 greedy decode, 80B-A3B-shaped Q4_K hybrid MoE", "host": "cpu"},
                    "cpu_baseline": cb, "e2e": {"value": cb["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                    "parity": parity}
            print(json.dumps(line))
        return

    # every rank holds the whole checkpoint; the headline step is one sequence per rank, the 64-slot measurement splits
    # its slots over the ranks and (second arm) shards the routed experts with exchanges over NVLink peer memory
    t0 = time.time()
    model = pkg.Model.synthetic(cfg, seed=0, device=local_rank)
    t_model = time.time() - t0
    if args.profile_prefill:
        n = args.profile_prefill
        gp = pkg.Graph(model, n_kv=2 * n + 64, max_tokens=n, slots=1, use_cuda_graph=False)
        ids = np.random.default_rng(1).integers(0, cfg["vocab"], 2 * n).astype(np.int32)
        gp.forward(ids[:n])
        torch.cuda.synchronize()
        torch.cuda.profiler.start()
        gp.extend(ids[n:])
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
        print(json.dumps({"profiled_prefill_rows": n}))
        return
    if args.profile_batch:
        gb = pkg.Graph(model, n_kv=32768 + 64, max_tokens=max(args.slots, 8), slots=args.slots, use_cuda_graph=False)
        rng_b = np.random.default_rng(7)   # the contexts and first tokens of batched_decode (rank 0)
        ctx = rng_b.integers(8192, 32769, args.slots)
        for s_ in range(args.slots):
            gb.use_slot(s_); gb.synth_context(int(ctx[s_]), seed=1000 + s_)
        sl = list(range(args.slots))
        # distinct random first tokens: identical rows would all select the same ten experts
        out = gb.generate_greedy(sl, rng_b.integers(0, cfg["vocab"], args.slots).astype(np.int32), 2)
        torch.cuda.synchronize()
        torch.cuda.profiler.start()
        out = gb.generate_greedy(sl, out[-1], args.profile_batch)
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
        print(json.dumps({"profiled_batch_steps": args.profile_batch, "slots": args.slots}))
        return
    n_kv = prompt_len + 2 * (steps + warmup) + 64
    g = pkg.Graph(model, n_kv=n_kv, max_tokens=args.chunk, slots=1, use_cuda_graph=not args.profile)
    rng = np.random.default_rng(1 + rank)
    prompt = rng.integers(0, cfg["vocab"], prompt_len).astype(np.int32)
    g.forward(prompt[:min(prompt_len, args.chunk)])   # first-use set-up of the many-row kernels, untimed
    torch.cuda.synchronize()
    t0 = time.time()
    logits, _ = g.forward(prompt)
    t_prefill = time.time() - t0
    tok = int(np.argmax(logits))

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    if args.profile:
        for _ in range(3):
            logits, _ = g.extend([tok]); tok = int(np.argmax(logits))
        torch.cuda.synchronize()
        torch.cuda.profiler.start()
        for _ in range(args.profile):
            logits, _ = g.extend([tok]); tok = int(np.argmax(logits))
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
        print(json.dumps({"profiled_steps": args.profile, "context": g.past()}))
        return
    # ---- device-resident loop: `value` ----
    out = g.generate_greedy([0], [tok], warmup)
    tok = int(out[-1, 0])
    ctx0 = g.past()
    barrier()
    with ClockSampler(local_rank) as clocks:
        out = g.generate_greedy([0], [tok], steps)
        barrier()
    dev_ms = g.last_device_ms()
    launches = g.last_launches()
    tok = int(out[-1, 0])
    dev_ms = max_over_ranks(dev_ms, world)
    # ---- end to end through the reference-facing call: id in, logits out, host argmax ----
    for _ in range(3):
        logits, _ = g.extend([tok]); tok = int(np.argmax(logits))
    barrier()
    e2e_steps = steps
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        logits, _ = g.extend([tok])
        tok = int(np.argmax(logits))
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    e2e_s = max_over_ranks(e2e_s, world)

    g.destroy()
    # ---- BASELINE config 3: 64 slots in all with 8k-32k contexts, split over the ranks (strong scaling) ----
    batch = None
    if args.slots > 0 and args.config == "a3b":
        try:
            batch = batched_decode(pkg, model, cfg, args.slots, min(steps, 32), rank, world, dist, barrier)
        except Exception as e:  # an extra measurement must not lose the headline line
            batch = {"error": str(e)[:300]}
    spec = config4 = None
    if rank == 0 and world == 1 and args.slots > 0 and args.config == "a3b":
        try:
            spec = verify_pass_times(pkg, model, cfg, prompt, torch)
            spec["batch1"] = speculative_decode(pkg, model, cfg, torch, 1, 4096, 48)
            spec["batch16"] = speculative_decode(pkg, model, cfg, torch, 16, 512, 16, depths=(2,))
        except Exception as e:  # an extra measurement must not lose the headline line
            spec = dict(spec or {}, error=str(e)[:300])
    if args.slots > 0 and args.config == "a3b":
        # config 4 on every rank: the prompt is one sequence and its attention / DeltaNet layers do not shard, so N GPUs
        # prefill N prompts (replicas); the slowest rank's time counts
        try:
            config4 = prefill_config4(pkg, model, cfg, torch)
            secs = max_over_ranks(config4["seconds"], world)
            config4.update(seconds=round(secs, 3), value=world * config4["prompt_tokens"] / secs, n_gpus=world,
                           parallelism="replicas: one prompt per GPU" if world > 1 else "single GPU")
        except Exception as e:
            config4 = {"error": str(e)[:300]}
    if rank == 0:
        ms_per_step = dev_ms / steps
        value = whole_job_rate(steps, world, dev_ms)
        bytes_step = algorithmic_bytes_per_token(pkg, cfg, ctx0 + steps // 2)
        peak, which = measured_peak_gbs()
        achieved = bytes_step / (ms_per_step / 1e3) / 1e9
        line = {
            "metric": METRIC, "value": value, "unit": "tok/s", "n_gpus": world, "steps": steps, "warmup": warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": f"batch-1 greedy decode after a {prompt_len}-token random prompt, {cfg['name']} "
                                   "(48 layers: 36 gated DeltaNet + 12 gated GQA, 512 experts top-10 + shared, Q4_K experts, "
                                   "Q5_K/Q6_K projections, Q8_0 router, Q6_K head), fp16 KV cache" if args.config == "a3b" else cfg["name"],
                       "context": ctx0, "weights_gb": model.weight_bytes / 1e9, "l2_policy": "inputs larger than L2 (2.5 GB streamed per step)",
                       "parallelism": "replicas (headline); batch64: 64 slots split over the ranks, slot_split and expert_parallel arms" if world > 1 else "single GPU", "model_build_s": round(t_model, 1),
                       "prefill_s": round(t_prefill, 3), "prefill_tok_s": round(prompt_len / t_prefill, 1), "prefill_chunk": args.chunk},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": A3B_DRAM_BYTES_PER_STEP if args.config == "a3b" and not args.layers else None,
                         "peak_source": which, "kernel": "one decode step (CUDA graph of the token loop)",
                         "algorithmic_bytes_per_step": bytes_step},
            "e2e": {"value": world * e2e_steps / e2e_s, "unit": "tok/s", "h2d_bytes_per_step": 4 + 16 + 16,
                    "d2h_bytes_per_step": cfg["vocab"] * 4 + cfg["n_embd"] * 4},
            "gpu_launches": launches * steps,
            "clocks": clocks.summary(),
        }
        if spec is not None:
            line["spec"] = spec
        if config4 is not None:
            line["prefill_32k"] = config4
        if batch is not None:
            line["batch64"] = batch
        if not args.no_cpu_baseline and world == 1:
            try:
                line["cpu_baseline"], line["parity"] = cpu_baseline(pkg, cfg, local_rank)
            except Exception as e:  # the baseline is a reported number, never a reason to lose the line
                line["cpu_baseline"] = {"value": None, "unit": "tok/s", "cores": 0, "kind": "port", "sample": f"failed: {e}"}
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
