"""Model shapes and the tensor manifest of a hybrid DeltaNet / attention / MoE checkpoint.

Tensor names, layouts and metadata keys are the ones the reference's loader reads
(llm/model.go:66-96, 375-468; llm/moe.go:136-183; llm/mtp.go:36-48), plus the plain
pre-norm glue (`attn_norm`, `ffn_norm`, `output_norm`, `nextn.shared_head_norm`) that a
model without hyper-connections needs.
"""
import math

from . import gguf

# Every `full_attention_interval`-th layer is gated GQA attention, the rest gated DeltaNet.
TINY = dict(
    name="tiny-hybrid-moe", n_layer=4, full_attention_interval=4, n_embd=1024, vocab=32768,
    n_head=8, n_head_kv=2, head_dim=128, rope_dims=32, rope_base=1e7, eps=1e-6,
    n_expert=32, n_expert_used=4, ffn_expert=256, ffn_shared=256,
    dn_head_dim=128, dn_heads_k=8, dn_heads_v=16, dn_conv=4, has_draft=0,
    types=dict(expert=gguf.Q4_K, shared=gguf.Q4_K, dn=gguf.Q4_K, attn=gguf.Q4_K, attn_v=gguf.Q4_K,
               router=gguf.Q8_0, embd=gguf.Q6_K, head=gguf.Q6_K, eh_proj=gguf.Q4_K))

A3B = dict(
    name="80b-a3b-shaped", n_layer=48, full_attention_interval=4, n_embd=2048, vocab=151936,
    n_head=16, n_head_kv=2, head_dim=256, rope_dims=64, rope_base=1e7, eps=1e-6,
    n_expert=512, n_expert_used=10, ffn_expert=512, ffn_shared=512,
    dn_head_dim=128, dn_heads_k=16, dn_heads_v=32, dn_conv=4, has_draft=0,
    types=dict(expert=gguf.Q4_K, shared=gguf.Q4_K, dn=gguf.Q5_K, attn=gguf.Q5_K, attn_v=gguf.Q6_K,
               router=gguf.Q8_0, embd=gguf.Q6_K, head=gguf.Q6_K, eh_proj=gguf.Q5_K))

CONFIGS = {"tiny": TINY, "a3b": A3B}


def variant(base, **over):
    c = dict(base)
    c["types"] = dict(base["types"])
    for k, v in over.items():
        if k == "types":
            c["types"].update(v)
        else:
            c[k] = v
    return c


def is_attention_layer(cfg, l):
    return (l + 1) % cfg["full_attention_interval"] == 0


# Value rules for synthetic tensors: ("normal", mean, std) | ("neg_exp_uniform", lo, hi)
W = ("normal", 0.0, 0.02)
G = ("normal", 1.0, 0.01)
# Depthwise conv taps are O(1) in trained checkpoints. Drawn at 0.02 like the matrices they
# leave the delta-rule read-out at the level of the gated norm's epsilon, and the layer's
# output then depends on the order a dot product is summed in (the CPU oracle disagrees with
# itself by 20% on some tokens when only its summation order is reversed).
CONV = ("normal", 0.0, 0.5)


def _mixer_and_moe(cfg, l, attn):
    """(name, type, ggml dims, value rule) of one layer, in a fixed order."""
    H, t = cfg["n_embd"], cfg["types"]
    p = f"blk.{l}."
    out = [(p + "attn_norm.weight", gguf.F32, (H,), G)]
    if attn:
        hd, nh, nkv = cfg["head_dim"], cfg["n_head"], cfg["n_head_kv"]
        out += [
            (p + "attn_q.weight", t["attn"], (H, nh * 2 * hd), W),      # per head: hd query rows then hd gate rows
            (p + "attn_k.weight", t["attn"], (H, nkv * hd), W),
            (p + "attn_v.weight", t["attn_v"], (H, nkv * hd), W),
            (p + "attn_q_norm.weight", gguf.F32, (hd,), G),
            (p + "attn_k_norm.weight", gguf.F32, (hd,), G),
            (p + "attn_output.weight", t["attn"], (nh * hd, H), W),
        ]
    else:
        d, hk, hv, K = cfg["dn_head_dim"], cfg["dn_heads_k"], cfg["dn_heads_v"], cfg["dn_conv"]
        cw = (2 * hk + hv) * d
        out += [
            (p + "attn_qkv.weight", t["dn"], (H, cw), W),               # q heads | k heads | v heads (tiled order)
            (p + "attn_gate.weight", t["dn"], (H, hv * d), W),
            (p + "ssm_alpha.weight", gguf.F32, (H, hv), W),
            (p + "ssm_beta.weight", gguf.F32, (H, hv), W),
            (p + "ssm_conv1d.weight", gguf.F32, (K, cw), CONV),            # taps of one channel contiguous
            (p + "ssm_a", gguf.F32, (hv,), ("neg_exp_uniform", 0.0, math.log(16.0))),  # -exp(A_log)
            (p + "ssm_dt.bias", gguf.F32, (hv,), W),
            (p + "ssm_norm.weight", gguf.F32, (d,), G),
            (p + "ssm_out.weight", t["dn"], (hv * d, H), W),
        ]
    nE, ff, ffs = cfg["n_expert"], cfg["ffn_expert"], cfg["ffn_shared"]
    out += [
        (p + "ffn_norm.weight", gguf.F32, (H,), G),
        (p + "ffn_gate_inp.weight", t["router"], (H, nE), W),
        (p + "ffn_gate_inp_shexp.weight", gguf.F32, (H,), W),
        (p + "ffn_gate_exps.weight", t["expert"], (H, ff, nE), W),      # expert e's row j is row e*ff + j
        (p + "ffn_up_exps.weight", t["expert"], (H, ff, nE), W),
        (p + "ffn_down_exps.weight", t["expert"], (ff, H, nE), W),
        (p + "ffn_gate_shexp.weight", t["shared"], (H, ffs), W),
        (p + "ffn_up_shexp.weight", t["shared"], (H, ffs), W),
        (p + "ffn_down_shexp.weight", t["shared"], (ffs, H), W),
    ]
    return out


def manifest(cfg):
    """Every tensor of the checkpoint as (name, ggml type, ggml dims, value rule), in draw order."""
    H, V, t = cfg["n_embd"], cfg["vocab"], cfg["types"]
    out = [("token_embd.weight", t["embd"], (H, V), W)]
    for l in range(cfg["n_layer"]):
        out += _mixer_and_moe(cfg, l, is_attention_layer(cfg, l))
    out += [("output_norm.weight", gguf.F32, (H,), G), ("output.weight", t["head"], (H, V), W)]
    if cfg.get("has_draft"):
        L = cfg["n_layer"]
        p = f"blk.{L}."
        out += _mixer_and_moe(cfg, L, True)
        out += [(p + "nextn.enorm.weight", gguf.F32, (H,), G), (p + "nextn.hnorm.weight", gguf.F32, (H,), G),
                (p + "nextn.eh_proj.weight", t["eh_proj"], (2 * H, H), W),
                (p + "nextn.shared_head_norm.weight", gguf.F32, (H,), G)]
    return out


def metadata(cfg, arch="qwen3next"):
    """(key, tag, value[, element tag]) rows for the GGUF header."""
    a = arch + "."
    half = cfg["rope_dims"] // 2
    s0 = (half + 2) // 3
    s1 = (half + 1) // 3
    sections = [s0, s1, half - s0 - s1, 0]  # covers every rotary pair, so text positions are plain NeoX
    return [
        (a + "block_count", gguf.U32, cfg["n_layer"] + (1 if cfg.get("has_draft") else 0)),
        (a + "nextn_predict_layers", gguf.U32, 1 if cfg.get("has_draft") else 0),
        (a + "embedding_length", gguf.U32, cfg["n_embd"]),
        (a + "attention.head_count", gguf.U32, cfg["n_head"]),
        (a + "attention.head_count_kv", gguf.U32, cfg["n_head_kv"]),
        (a + "attention.key_length", gguf.U32, cfg["head_dim"]),
        (a + "attention.layer_norm_rms_epsilon", gguf.FLT32, cfg["eps"]),
        (a + "rope.dimension_count", gguf.U32, cfg["rope_dims"]),
        (a + "rope.freq_base", gguf.FLT32, cfg["rope_base"]),
        (a + "rope.dimension_sections", gguf.ARR, sections, gguf.I32),
        (a + "expert_count", gguf.U32, cfg["n_expert"]),
        (a + "expert_used_count", gguf.U32, cfg["n_expert_used"]),
        (a + "expert_feed_forward_length", gguf.U32, cfg["ffn_expert"]),
        (a + "expert_shared_feed_forward_length", gguf.U32, cfg["ffn_shared"]),
        (a + "ssm.state_size", gguf.U32, cfg["dn_head_dim"]),
        (a + "ssm.group_count", gguf.U32, cfg["dn_heads_k"]),
        (a + "ssm.time_step_rank", gguf.U32, cfg["dn_heads_v"]),
        (a + "ssm.conv_kernel", gguf.U32, cfg["dn_conv"]),
        (a + "ssm.inner_size", gguf.U32, cfg["dn_heads_v"] * cfg["dn_head_dim"]),
        (a + "full_attention_interval", gguf.U32, cfg["full_attention_interval"]),
    ]


def graph_fields(cfg):
    keys = ("n_layer", "n_embd", "vocab", "n_head", "n_head_kv", "head_dim", "rope_dims", "rope_base", "eps", "n_expert",
            "n_expert_used", "ffn_expert", "ffn_shared", "dn_head_dim", "dn_heads_k", "dn_heads_v", "dn_conv", "has_draft")
    return {k: cfg[k] for k in keys}


def weight_bytes(cfg):
    """Bytes of every tensor in the manifest (a checkpoint's size on the device)."""
    return sum(gguf.tensor_bytes(t, d) for _, t, d, _ in manifest(cfg))
