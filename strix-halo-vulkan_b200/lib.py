"""ctypes binding of libb200llm.so (include/b200_llm.h). Loading fails loudly: there is no
CPU path behind this module."""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libb200llm.so")
_lib = None

OK, EINVAL, ECAPACITY, ECUDA, ENCCL, ETIMEOUT, ESTATE, ENOMEM, EIO = range(9)
STATUS_NAME = ["OK", "EINVAL", "ECAPACITY", "ECUDA", "ENCCL", "ETIMEOUT", "ESTATE", "ENOMEM", "EIO"]


# B200_W16_*: weight matrices a pass multiplies rounded to fp16 (b200_graph_fp16_weight_mask)
W16_DN_QKV, W16_DN_GATE, W16_DN_OUT, W16_ATTN_Q, W16_ATTN_K, W16_ATTN_V, W16_ATTN_OUT, W16_ROUTER, W16_EXPERTS, W16_SHARED, W16_HEAD = \
    (1 << b for b in range(8, 19))


class Config(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("n_layer", "n_embd", "vocab", "n_head", "n_head_kv", "head_dim", "rope_dims")] + \
               [("rope_base", C.c_float), ("eps", C.c_float)] + \
               [(n, C.c_int32) for n in ("n_expert", "n_expert_used", "ffn_expert", "ffn_shared", "dn_head_dim",
                                         "dn_heads_k", "dn_heads_v", "dn_conv", "has_draft")]


class GraphOpts(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("max_tokens", "n_kv", "slots", "speculative", "spec_rows", "attn_split_cells",
                                         "use_cuda_graph", "trace")]


class GraphStats(C.Structure):
    _fields_ = [("passes", C.c_int64), ("rows", C.c_int64), ("launches", C.c_int64), ("device_ms", C.c_double), ("host_ms", C.c_double),
                ("last_rows", C.c_int32), ("last_launches", C.c_int32), ("last_device_ms", C.c_float), ("expert_streams", C.c_int64)]


class EpHandle(C.Structure):
    _fields_ = [("bytes", C.c_ubyte * 64)]


class Input(C.Structure):
    _fields_ = [("ids", C.c_void_p), ("n", C.c_int32), ("n_images", C.c_int32)]


class B200Error(RuntimeError):
    def __init__(self, status, msg):
        super().__init__(f"{STATUS_NAME[status] if 0 <= status < len(STATUS_NAME) else status}: {msg}")
        self.status = status


# every exported symbol of include/b200_llm.h: name -> (restype, argtypes)
P, I32, I64, U32, U64, F32 = C.c_void_p, C.c_int32, C.c_int64, C.c_uint32, C.c_uint64, C.c_float
PP = C.POINTER(C.c_void_p)
SYMBOLS = {
    "b200_last_error": (C.c_char_p, []),
    "b200_device_count": (I32, []),
    "b200_model_new": (I32, [C.POINTER(Config), I32, PP]),
    "b200_model_add_tensor": (I32, [P, C.c_char_p, U32, U32, C.POINTER(I64), P]),
    "b200_model_add_synthetic": (I32, [P, C.c_char_p, U32, U32, C.POINTER(I64), U64, I32, F32, F32]),
    "b200_model_finalize": (I32, [P]),
    "b200_model_open_gguf": (I32, [C.c_char_p, I32, PP]),
    "b200_model_config": (I32, [P, C.POINTER(Config)]),
    "b200_model_weight_bytes": (I64, [P]),
    "b200_model_tensor_bytes": (I64, [P, C.c_char_p]),
    "b200_model_read_tensor": (I32, [P, C.c_char_p, P, I64]),
    "b200_model_free": (None, [P]),
    "b200_graph_create": (I32, [P, C.POINTER(GraphOpts), PP]),
    "b200_graph_destroy": (None, [P]),
    "b200_graph_slots": (I32, [P]),
    "b200_graph_nkv": (I32, [P]),
    "b200_graph_use_slot": (I32, [P, I32]),
    "b200_graph_reset": (I32, [P]),
    "b200_graph_past": (I32, [P]),
    "b200_graph_set_past": (I32, [P, I32]),
    "b200_graph_forward": (I32, [P, P, I32, PP, PP]),
    "b200_graph_extend": (I32, [P, P, I32, PP, PP]),
    "b200_graph_extend_input": (I32, [P, C.POINTER(Input), PP, PP]),
    "b200_graph_extend_rows": (I32, [P, P, I32, PP, PP]),
    "b200_graph_extend_residual": (I32, [P, P, I32, PP, PP]),
    "b200_graph_decode_rows": (I32, [P, P, P, I32, PP]),
    "b200_graph_checkpoint": (I32, [P, C.POINTER(I32)]),
    "b200_graph_restore": (I32, [P, I32]),
    "b200_graph_checkpoint_free": (I32, [P, I32]),
    "b200_graph_speculate": (I32, [P, I32]),
    "b200_graph_speculating": (I32, [P]),
    "b200_graph_speculate_first": (I32, [P, I32]),
    "b200_graph_keep": (I32, [P, I32]),
    "b200_graph_keep_first": (I32, [P]),
    "b200_graph_residual_row": (I32, [P, I32, P]),
    "b200_graph_pass_experts": (I32, [P, C.POINTER(I32)]),
    "b200_graph_fp16_weight_mask": (U32, [P, I32, I32]),
    "b200_graph_stats_get": (I32, [P, C.POINTER(GraphStats)]),
    "b200_graph_stats_reset": (I32, [P]),
    "b200_graph_inject_wait_timeout": (I32, [P]),
    "b200_graph_commit": (I32, [P]),
    "b200_graph_rewind": (I32, [P]),
    "b200_graph_ep_export": (I32, [P, I32, I32, C.POINTER(EpHandle)]),
    "b200_graph_ep_attach": (I32, [P, C.POINTER(EpHandle)]),
    "b200_graph_ep_prepare": (I32, [P, I32, I32]),
    "b200_graph_ep_attach_local": (I32, [P, PP, I32]),
    "b200_graph_ep_enable": (I32, [P, I32]),
    "b200_graph_synth_context": (I32, [P, I32, U64]),
    "b200_graph_generate_greedy": (I32, [P, P, P, I32, I32, P]),
    "b200_graph_last_device_ms": (F32, [P]),
    "b200_graph_last_launches": (I32, [P]),
    "b200_graph_timeline": (I32, [P, P, I32]),
    "b200_graph_trace": (I64, [P, I32, P, I64]),
    "b200_draft_rows": (I32, [P, P, P, I32, I32, PP, PP]),
    "b200_draft_set_vocab": (I32, [P, I32]),
    "b200_draft_use_slot": (I32, [P, I32]),
    "b200_draft_slots": (I32, [P]),
    "b200_draft_reset": (I32, [P]),
    "b200_draft_max_rows": (I32, [P]),
    "b200_draft_wide": (I32, [P]),
    "b200_draft_past": (I32, [P]),
    "b200_draft_rewind": (I32, [P, I32]),
    "b200_dequantize": (I32, [U32, P, I64, P]),
    "b200_qgemv": (I32, [U32, P, I64, I64, P, I32, P]),
    "b200_qgemv_static": (I32, [U32, P, I64, I64, P, I32, P]),
    "b200_qgemm": (I32, [U32, P, I64, I64, P, I32, I32, P]),
    "b200_quantize": (I32, [U32, P, I64, I64, P]),
}


def load():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: build it with `python strix-halo-vulkan_b200/build.py` "
                              "(the CUDA library is the only implementation; there is no fallback)")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(L, name)
            fn.restype, fn.argtypes = res, args
        _lib = L
    return _lib


def check(status):
    if status != OK:
        raise B200Error(status, load().b200_last_error().decode(errors="replace"))
