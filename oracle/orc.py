"""TEST INFRASTRUCTURE: ctypes binding of the CPU oracle (oracle/liboracle.so).

Only tests, the smoke check and the benchmark's cpu-baseline leg may import this module;
the product never does. The library is built by `make -C oracle`.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

EXACT, DEVICE_LIKE = 0, 1
# OR-ed into `numerics`: weight matrices rounded to fp16 after dequantisation (oracle.h ORC_W16_*)
W16_DN_QKV, W16_DN_GATE, W16_DN_OUT, W16_ATTN_Q, W16_ATTN_K, W16_ATTN_V, W16_ATTN_OUT, W16_ROUTER, W16_EXPERTS, W16_SHARED, W16_HEAD = \
    (1 << b for b in range(8, 19))
W16_ALL = sum(1 << b for b in range(8, 19))


class Tensor(C.Structure):
    _fields_ = [("name", C.c_char_p), ("type", C.c_uint32), ("n_dims", C.c_uint32),
                ("dims", C.c_int64 * 4), ("data", C.c_void_p)]


class Config(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("n_layer", "n_embd", "vocab", "n_head", "n_head_kv", "head_dim", "rope_dims")] + \
               [("rope_base", C.c_float), ("eps", C.c_float)] + \
               [(n, C.c_int32) for n in ("n_expert", "n_expert_used", "ffn_expert", "ffn_shared", "dn_head_dim",
                                         "dn_heads_k", "dn_heads_v", "dn_conv", "has_draft")]


class Trace(C.Structure):
    _fields_ = [("mix_out", C.c_void_p), ("ffn_out", C.c_void_p), ("hidden", C.c_void_p), ("normed", C.c_void_p),
                ("topk", C.c_void_p), ("topk_w", C.c_void_p), ("margin", C.c_void_p), ("logits", C.c_void_p), ("force_topk", C.c_void_p)]


def build(force=False):
    so = os.path.join(_HERE, "liboracle.so")
    srcs = [os.path.join(_HERE, f) for f in ("oracle.cpp", "oracle.h", "oracle_quant.h")]
    if force or not os.path.exists(so) or any(os.path.getmtime(s) > os.path.getmtime(so) for s in srcs):
        subprocess.check_call(["make", "-C", _HERE, "liboracle.so"], stdout=subprocess.DEVNULL)
    return so


def lib():
    global _LIB
    if _LIB is None:
        so = os.path.join(_HERE, "liboracle.so")
        if not os.path.exists(so):
            build()
        L = C.CDLL(so)
        L.orc_f32_to_f16.restype = C.c_uint16; L.orc_f32_to_f16.argtypes = [C.c_float]
        L.orc_f16_to_f32.restype = C.c_float; L.orc_f16_to_f32.argtypes = [C.c_uint16]
        L.orc_row_bytes.restype = C.c_int64; L.orc_row_bytes.argtypes = [C.c_uint32, C.c_int64]
        L.orc_dequantize.argtypes = [C.c_uint32, C.c_void_p, C.c_int64, C.c_void_p]
        L.orc_dequantize_w16.argtypes = [C.c_uint32, C.c_void_p, C.c_int64, C.c_void_p]
        L.orc_quantize.argtypes = [C.c_uint32, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p]
        L.orc_matvec.argtypes = [C.c_uint32, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p]
        L.orc_rmsnorm.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_float, C.c_void_p]
        L.orc_argmax.restype = C.c_int32; L.orc_argmax.argtypes = [C.c_void_p, C.c_int64]
        L.orc_model_create.restype = C.c_void_p
        L.orc_model_create.argtypes = [C.POINTER(Config), C.POINTER(Tensor), C.c_int, C.c_char_p, C.c_int]
        L.orc_model_destroy.argtypes = [C.c_void_p]
        L.orc_seq_create.restype = C.c_void_p; L.orc_seq_create.argtypes = [C.c_void_p]
        L.orc_draft_seq_create.restype = C.c_void_p; L.orc_draft_seq_create.argtypes = [C.c_void_p]
        L.orc_seq_clone.restype = C.c_void_p; L.orc_seq_clone.argtypes = [C.c_void_p]
        L.orc_seq_destroy.argtypes = [C.c_void_p]
        L.orc_seq_past.restype = C.c_int32; L.orc_seq_past.argtypes = [C.c_void_p]
        L.orc_extend.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.POINTER(Trace)]
        L.orc_draft_step.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int, C.c_void_p, C.c_void_p, C.c_int32]
        _LIB = L
    return _LIB


def row_bytes(typ, n):
    return int(lib().orc_row_bytes(typ, n))


def dequantize(typ, data, n):
    buf = np.ascontiguousarray(np.frombuffer(data, dtype=np.uint8))
    out = np.empty(n, dtype=np.float32)
    if lib().orc_dequantize(typ, buf.ctypes.data, n, out.ctypes.data) != 0:
        raise ValueError(f"cannot dequantize type {typ} x {n}")
    return out


def dequantize_w16(typ, data, n):
    """The elements as the tensor-core kernels multiply them (fp16 values)."""
    buf = np.ascontiguousarray(np.frombuffer(data, dtype=np.uint8))
    out = np.empty(n, dtype=np.float32)
    if lib().orc_dequantize_w16(typ, buf.ctypes.data, n, out.ctypes.data) != 0:
        raise ValueError(f"cannot dequantize type {typ} x {n}")
    return out


def quantize(typ, x):
    """x: [rows, k] float32 -> uint8 array of packed blocks."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    rows, k = (1, x.shape[0]) if x.ndim == 1 else (int(np.prod(x.shape[:-1])), x.shape[-1])
    rb = row_bytes(typ, k)
    if rb < 0:
        raise ValueError(f"type {typ} cannot hold rows of {k}")
    out = np.empty(rows * rb, dtype=np.uint8)
    if lib().orc_quantize(typ, x.ctypes.data, rows, k, out.ctypes.data) != 0:
        raise ValueError(f"cannot quantize to type {typ}")
    return out


def matvec(typ, w, rows, k, x):
    w = np.ascontiguousarray(np.frombuffer(w, dtype=np.uint8))
    x = np.ascontiguousarray(x, dtype=np.float32)
    y = np.empty(rows, dtype=np.float32)
    if lib().orc_matvec(typ, w.ctypes.data, rows, k, x.ctypes.data, y.ctypes.data) != 0:
        raise ValueError("matvec")
    return y


def rmsnorm(x, gamma, eps):
    x = np.ascontiguousarray(x, dtype=np.float32); gamma = np.ascontiguousarray(gamma, dtype=np.float32)
    out = np.empty_like(x)
    lib().orc_rmsnorm(x.ctypes.data, gamma.ctypes.data, x.size, eps, out.ctypes.data)
    return out


def argmax(logits):
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    return int(lib().orc_argmax(logits.ctypes.data, logits.size))


class Model:
    """cfg: dict with the Config field names; tensors: {name: (type, dims(ggml order), uint8 ndarray)}."""

    def __init__(self, cfg, tensors):
        self.cfg = Config(**{k: v for k, v in cfg.items() if k in dict(Config._fields_)})
        self._keep = []
        arr = (Tensor * len(tensors))()
        for i, (name, (typ, dims, data)) in enumerate(tensors.items()):
            data = np.ascontiguousarray(data)
            self._keep.append(data)
            arr[i].name = name.encode(); arr[i].type = typ; arr[i].n_dims = len(dims)
            for d in range(4):
                arr[i].dims[d] = dims[d] if d < len(dims) else 1
            arr[i].data = data.ctypes.data
        err = C.create_string_buffer(512)
        self.h = lib().orc_model_create(C.byref(self.cfg), arr, len(tensors), err, 512)
        if not self.h:
            raise ValueError("oracle model: " + err.value.decode())

    def __del__(self):
        if getattr(self, "h", None):
            lib().orc_model_destroy(self.h); self.h = None

    def seq(self):
        return Seq(self, lib().orc_seq_create(self.h))

    def draft_seq(self):
        return Seq(self, lib().orc_draft_seq_create(self.h))


class Seq:
    def __init__(self, model, h):
        self.model, self.h = model, h

    def __del__(self):
        if getattr(self, "h", None):
            lib().orc_seq_destroy(self.h); self.h = None

    def clone(self):
        return Seq(self.model, lib().orc_seq_clone(self.h))

    @property
    def past(self):
        return int(lib().orc_seq_past(self.h))

    def extend(self, ids, numerics=DEVICE_LIKE, trace=(), want_last=True, force_topk=None):
        """Advance by len(ids) tokens. Returns (last-row logits or None, {trace name: array}). force_topk
        [n][n_layer][used] (int32, rows < 0: own choice) makes the MoE blocks route to the given experts in that slot
        order; the trace's topk / margin still report the oracle's own selection."""
        c = self.model.cfg
        ids = np.ascontiguousarray(ids, dtype=np.int32)
        n = ids.size
        H, nl, used, V = c.n_embd, c.n_layer, c.n_expert_used, c.vocab
        shapes = {"mix_out": ((n, nl, H), np.float32), "ffn_out": ((n, nl, H), np.float32), "hidden": ((n, nl, H), np.float32),
                  "normed": ((n, H), np.float32), "topk": ((n, nl, used), np.int32), "topk_w": ((n, nl, used), np.float32),
                  "margin": ((n, nl), np.float32), "logits": ((n, V), np.float32)}
        out, tr = {}, Trace()
        for name in trace:
            shp, dt = shapes[name]
            out[name] = np.zeros(shp, dtype=dt)
            setattr(tr, name, out[name].ctypes.data)
        if force_topk is not None:
            forced = np.ascontiguousarray(force_topk, dtype=np.int32)
            if forced.shape != (n, nl, used):
                raise ValueError(f"force_topk must be {(n, nl, used)}, got {forced.shape}")
            tr.force_topk = forced.ctypes.data
        last = np.empty(V, dtype=np.float32) if want_last else None
        rc = lib().orc_extend(self.model.h, self.h, ids.ctypes.data, n, numerics,
                              last.ctypes.data if want_last else None, C.byref(tr))
        if rc != 0:
            raise ValueError(f"orc_extend failed: {rc}")
        return last, out

    def draft_step(self, h_prev, tok, numerics=DEVICE_LIKE, draft_vocab=0):
        c = self.model.cfg
        h_prev = np.ascontiguousarray(h_prev, dtype=np.float32)
        h_out = np.empty(c.n_embd, dtype=np.float32)
        nv = draft_vocab if 0 < draft_vocab < c.vocab else c.vocab
        logits = np.empty(nv, dtype=np.float32)
        rc = lib().orc_draft_step(self.model.h, self.h, h_prev.ctypes.data, int(tok), numerics,
                                  h_out.ctypes.data, logits.ctypes.data, draft_vocab)
        if rc != 0:
            raise ValueError(f"orc_draft_step failed: {rc}")
        return h_out, logits
