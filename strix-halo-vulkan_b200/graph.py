"""Host-side mirror of the reference's `llm.Graph` method set (llm/graph.go:184) over the
C ABI: the calls `backend/llm.go` and `backend/llm_sched.go` make, with the same names,
argument meaning and refusal behaviour. Returned arrays are copies of the library's pinned
buffers, so they stay valid across later calls."""
import ctypes as C

import numpy as np

from . import config as _config
from . import gguf as _gguf
from . import lib as _lib

RULES = {"normal": 0, "neg_exp_uniform": 1}


def _i32(a):
    return np.ascontiguousarray(a, dtype=np.int32)


class Model:
    """A checkpoint on one device. Build with `Model.open(path)`, `Model.from_tensors(cfg, tensors)`
    or `Model.synthetic(cfg, seed)`."""

    def __init__(self, handle, cfg):
        self._h, self.cfg = handle, cfg

    @classmethod
    def open(cls, path, device=0):
        L = _lib.load()
        h = C.c_void_p()
        _lib.check(L.b200_model_open_gguf(str(path).encode(), device, C.byref(h)))
        c = _lib.Config()
        _lib.check(L.b200_model_config(h, C.byref(c)))
        return cls(h, {n: getattr(c, n) for n, _ in _lib.Config._fields_})

    @classmethod
    def _new(cls, cfg, device):
        L = _lib.load()
        c = _lib.Config(**{k: cfg[k] for k, _ in _lib.Config._fields_})
        h = C.c_void_p()
        _lib.check(L.b200_model_new(C.byref(c), device, C.byref(h)))
        return cls(h, {k: cfg[k] for k, _ in _lib.Config._fields_})

    @classmethod
    def from_tensors(cls, cfg, tensors, device=0):
        """tensors: {name: (ggml type, ggml dims, uint8 array in GGUF block layout)}: what the
        Go host would pass from its mmap'd gguf.Tensor table."""
        m = cls._new(cfg, device)
        L = _lib.load()
        for name, (typ, dims, data) in tensors.items():
            data = np.ascontiguousarray(data)
            d = (C.c_int64 * len(dims))(*dims)
            _lib.check(L.b200_model_add_tensor(m._h, name.encode(), typ, len(dims), d, data.ctypes.data))
        _lib.check(L.b200_model_finalize(m._h))
        return m

    @classmethod
    def synthetic(cls, cfg, seed=0, device=0):
        """Every tensor of config.manifest(cfg) generated and quantised on the device."""
        m = cls._new(_config.graph_fields(cfg), device)
        L = _lib.load()
        for i, (name, typ, dims, (rule, p0, p1)) in enumerate(_config.manifest(cfg)):
            d = (C.c_int64 * len(dims))(*dims)
            _lib.check(L.b200_model_add_synthetic(m._h, name.encode(), typ, len(dims), d, seed * 1000003 + i, RULES[rule], p0, p1))
        _lib.check(L.b200_model_finalize(m._h))
        return m

    @property
    def weight_bytes(self):
        return int(_lib.load().b200_model_weight_bytes(self._h))

    def read_tensor(self, name):
        L = _lib.load()
        n = L.b200_model_tensor_bytes(self._h, name.encode())
        if n < 0:
            raise KeyError(name)
        out = np.empty(n, dtype=np.uint8)
        _lib.check(L.b200_model_read_tensor(self._h, name.encode(), out.ctypes.data, n))
        return out

    def close(self):
        if self._h:
            _lib.load().b200_model_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Graph:
    """llm.Graph: NewGraph(model, GraphOpts{MaxTokens, NKV, Slots, Speculative, SpecRows})."""

    def __init__(self, model, n_kv, max_tokens=64, slots=1, speculative=False, spec_rows=0, attn_split_cells=0,
                 use_cuda_graph=True, trace=False):
        self.model = model
        L = _lib.load()
        o = _lib.GraphOpts(max_tokens, n_kv, slots, int(speculative), spec_rows, attn_split_cells, int(use_cuda_graph), int(trace))
        self._h = C.c_void_p()
        _lib.check(L.b200_graph_create(model._h, C.byref(o), C.byref(self._h)))
        self.vocab, self.n_embd = model.cfg["vocab"], model.cfg["n_embd"]
        self.max_tokens = max_tokens
        self._draft_vocab = 0

    def destroy(self):
        if self._h:
            _lib.load().b200_graph_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass

    # -- slots ---------------------------------------------------------------------------
    def slots(self):
        return int(_lib.load().b200_graph_slots(self._h))

    def nkv(self):
        return int(_lib.load().b200_graph_nkv(self._h))

    def use_slot(self, s):
        _lib.check(_lib.load().b200_graph_use_slot(self._h, s))

    def reset(self):
        _lib.check(_lib.load().b200_graph_reset(self._h))

    def past(self):
        return int(_lib.load().b200_graph_past(self._h))

    def set_past(self, past):
        _lib.check(_lib.load().b200_graph_set_past(self._h, past))

    def synth_context(self, cells, seed=0):
        """Fills the current slot's caches and state with seeded values and declares `cells` cells prefilled."""
        _lib.check(_lib.load().b200_graph_synth_context(self._h, cells, seed))

    # -- expert parallelism ----------------------------------------------------------------
    def ep_export(self, rank, world):
        """This rank's exchange buffers as 64 opaque bytes for the other ranks' processes."""
        h = _lib.EpHandle()
        _lib.check(_lib.load().b200_graph_ep_export(self._h, rank, world, C.byref(h)))
        return bytes(h.bytes)

    def ep_attach(self, handles):
        arr = (_lib.EpHandle * len(handles))()
        for i, b in enumerate(handles):
            C.memmove(arr[i].bytes, bytes(b), 64)
        _lib.check(_lib.load().b200_graph_ep_attach(self._h, arr))

    @staticmethod
    def ep_connect_local(graphs):
        """Ranks in one process, one graph per device, in rank order."""
        L = _lib.load()
        n = len(graphs)
        for r, g in enumerate(graphs):
            _lib.check(L.b200_graph_ep_prepare(g._h, r, n))
        arr = (C.c_void_p * n)(*[g._h.value for g in graphs])
        for g in graphs:
            _lib.check(L.b200_graph_ep_attach_local(g._h, arr, n))

    def ep_enable(self, on=True):
        _lib.check(_lib.load().b200_graph_ep_enable(self._h, int(on)))

    # -- passes --------------------------------------------------------------------------
    def _call(self, fn, ids, rows_logits, rows_hidden, vocab=None):
        ids = _i32(ids)
        lg, hd = C.c_void_p(), C.c_void_p()
        _lib.check(fn(self._h, ids.ctypes.data, ids.size, C.byref(lg), C.byref(hd)))
        V = vocab or self.vocab
        logits = np.ctypeslib.as_array(C.cast(lg, C.POINTER(C.c_float)), (rows_logits, V)).copy()
        hidden = np.ctypeslib.as_array(C.cast(hd, C.POINTER(C.c_float)), (rows_hidden, self.n_embd)).copy()
        return logits, hidden

    def forward(self, ids):
        lg, hd = self._call(_lib.load().b200_graph_forward, ids, 1, 1)
        return lg[0], hd[0]

    def extend(self, ids):
        """(logits [vocab] of the last row, residual [n_embd] of the last row)."""
        lg, hd = self._call(_lib.load().b200_graph_extend, ids, 1, 1)
        return lg[0], hd[0]

    def extend_input(self, ids, n_images=0):
        """Graph.ExtendInput (llm/graph.go:1716); inputs that carry images are refused (no vision tower)."""
        ids = _i32(ids)
        inp = _lib.Input(ids.ctypes.data, ids.size, n_images)
        lg, hd = C.c_void_p(), C.c_void_p()
        _lib.check(_lib.load().b200_graph_extend_input(self._h, C.byref(inp), C.byref(lg), C.byref(hd)))
        return (np.ctypeslib.as_array(C.cast(lg, C.POINTER(C.c_float)), (self.vocab,)).copy(),
                np.ctypeslib.as_array(C.cast(hd, C.POINTER(C.c_float)), (self.n_embd,)).copy())

    def residual_row(self, r):
        out = np.empty(self.n_embd, dtype=np.float32)
        _lib.check(_lib.load().b200_graph_residual_row(self._h, r, out.ctypes.data))
        return out

    def pass_experts(self):
        n = C.c_int32()
        _lib.check(_lib.load().b200_graph_pass_experts(self._h, C.byref(n)))
        return n.value

    def fp16_weight_mask(self, rows, logit_rows=1):
        """B200_W16_* bits: the weight matrices a pass of `rows` rows multiplies rounded to fp16 (tensor-core kernels)."""
        return int(_lib.load().b200_graph_fp16_weight_mask(self._h, rows, logit_rows))

    def stats(self):
        st = _lib.GraphStats()
        _lib.check(_lib.load().b200_graph_stats_get(self._h, C.byref(st)))
        return {n: getattr(st, n) for n, _ in _lib.GraphStats._fields_}

    def stats_reset(self):
        _lib.check(_lib.load().b200_graph_stats_reset(self._h))

    def inject_wait_timeout(self):
        """Queues a kernel whose bounded wait must run out: the next pass reports ETIMEOUT (nothing faults)."""
        _lib.check(_lib.load().b200_graph_inject_wait_timeout(self._h))

    def extend_rows(self, ids):
        n = len(ids)
        return self._call(_lib.load().b200_graph_extend_rows, ids, n, n)

    def extend_residual(self, ids):
        lg, res = self._call(_lib.load().b200_graph_extend_residual, ids, 1, len(ids))
        return lg[0], res

    def decode_rows(self, slots, ids):
        slots, ids = _i32(slots), _i32(ids)
        if slots.size != ids.size:
            raise ValueError("decode_rows: one id per slot")
        lg = C.c_void_p()
        _lib.check(_lib.load().b200_graph_decode_rows(self._h, slots.ctypes.data, ids.ctypes.data, ids.size, C.byref(lg)))
        return np.ctypeslib.as_array(C.cast(lg, C.POINTER(C.c_float)), (ids.size, self.vocab)).copy()

    def generate_greedy(self, slots, first_ids, steps):
        """Device-resident greedy loop: returns ids [steps][n]; only ids cross the bus."""
        slots, first = _i32(slots), _i32(first_ids)
        out = np.empty((steps, slots.size), dtype=np.int32)
        _lib.check(_lib.load().b200_graph_generate_greedy(self._h, slots.ctypes.data, first.ctypes.data, slots.size, steps, out.ctypes.data))
        return out

    def last_device_ms(self):
        return float(_lib.load().b200_graph_last_device_ms(self._h))

    def last_launches(self):
        return int(_lib.load().b200_graph_last_launches(self._h))

    # -- sequence checkpoints and speculation -----------------------------------------------
    def checkpoint(self):
        h = C.c_int32()
        _lib.check(_lib.load().b200_graph_checkpoint(self._h, C.byref(h)))
        return h.value

    def restore(self, handle):
        _lib.check(_lib.load().b200_graph_restore(self._h, handle))

    def checkpoint_free(self, handle):
        _lib.check(_lib.load().b200_graph_checkpoint_free(self._h, handle))

    def speculate(self, on):
        _lib.check(_lib.load().b200_graph_speculate(self._h, int(on)))

    def speculating(self):
        return bool(_lib.load().b200_graph_speculating(self._h))

    def speculate_first(self, on):
        _lib.check(_lib.load().b200_graph_speculate_first(self._h, int(on)))

    def keep_first(self):
        _lib.check(_lib.load().b200_graph_keep_first(self._h))

    def keep(self, k):
        _lib.check(_lib.load().b200_graph_keep(self._h, k))

    def commit(self):
        _lib.check(_lib.load().b200_graph_commit(self._h))

    def rewind(self):
        _lib.check(_lib.load().b200_graph_rewind(self._h))

    # -- draft head ---------------------------------------------------------------------------
    def draft_rows(self, hs, ids, vocab_k=0):
        hs = np.ascontiguousarray(hs, dtype=np.float32).reshape(-1, self.n_embd)
        ids = _i32(ids)
        res, lg = C.c_void_p(), C.c_void_p()
        _lib.check(_lib.load().b200_draft_rows(self._h, hs.ctypes.data, ids.ctypes.data, ids.size, vocab_k, C.byref(res), C.byref(lg)))
        vocab_k = vocab_k or self._draft_vocab
        V = vocab_k if 0 < vocab_k < self.vocab else self.vocab
        return (np.ctypeslib.as_array(C.cast(res, C.POINTER(C.c_float)), (ids.size, self.n_embd)).copy(),
                np.ctypeslib.as_array(C.cast(lg, C.POINTER(C.c_float)), (ids.size, V)).copy())

    def draft_set_vocab(self, k):
        _lib.check(_lib.load().b200_draft_set_vocab(self._h, k))
        self._draft_vocab = 0 if k == self.vocab else k

    def draft_use_slot(self, s):
        _lib.check(_lib.load().b200_draft_use_slot(self._h, s))

    def draft_slots(self):
        return int(_lib.load().b200_draft_slots(self._h))

    def draft_reset(self):
        _lib.check(_lib.load().b200_draft_reset(self._h))

    def draft_max_rows(self):
        return int(_lib.load().b200_draft_max_rows(self._h))

    def draft_wide(self):
        return int(_lib.load().b200_draft_wide(self._h))

    def draft_past(self):
        return int(_lib.load().b200_draft_past(self._h))

    def draft_rewind(self, past):
        _lib.check(_lib.load().b200_draft_rewind(self._h, past))

    def timeline(self, max_launches=1024):
        """[launches][8] globaltimer ns of the last pass (process started with B200_TIMELINE=1)."""
        a = np.zeros((max_launches, 8), dtype=np.int64)
        n = _lib.load().b200_graph_timeline(self._h, a.ctypes.data, max_launches)
        return a[:max(n, 0)]

    # -- trace --------------------------------------------------------------------------------
    def trace(self, rows):
        """Per-layer tensors of the last pass (graph created with trace=True)."""
        c = self.model.cfg
        nl, H, used = c["n_layer"], c["n_embd"], c["n_expert_used"]
        L = _lib.load()
        out = {}
        for what, name, shape, dt in ((0, "after_mixer", (nl, rows, H), np.float32), (1, "hidden", (nl, rows, H), np.float32),
                                      (2, "topk", (nl, rows, used), np.int32), (3, "topk_w", (nl, rows, used + 1), np.float32),
                                      (4, "margin", (nl, rows), np.float32)):
            a = np.empty(shape, dtype=dt)
            n = L.b200_graph_trace(self._h, what, a.ctypes.data, a.nbytes)
            if n < 0:
                _lib.check(int(-n))
            out[name] = a
        return out


# -- unit entry points ----------------------------------------------------------------------
def dequantize(typ, data, n):
    data = np.ascontiguousarray(np.frombuffer(data, dtype=np.uint8))
    out = np.empty(n, dtype=np.float32)
    _lib.check(_lib.load().b200_dequantize(typ, data.ctypes.data, n, out.ctypes.data))
    return out


def qgemv(typ, w, rows, k, x):
    w = np.ascontiguousarray(np.frombuffer(w, dtype=np.uint8))
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, k)
    y = np.empty((x.shape[0], rows), dtype=np.float32)
    _lib.check(_lib.load().b200_qgemv(typ, w.ctypes.data, rows, k, x.ctypes.data, x.shape[0], y.ctypes.data))
    return y


def qgemm(typ, w, rows, k, x, tile_rows=64):
    """Many-row projection through the tensor-core kernel (weights rounded to fp16 after dequantisation)."""
    w = np.ascontiguousarray(np.frombuffer(w, dtype=np.uint8))
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, k)
    y = np.empty((x.shape[0], rows), dtype=np.float32)
    _lib.check(_lib.load().b200_qgemm(typ, w.ctypes.data, rows, k, x.ctypes.data, x.shape[0], tile_rows, y.ctypes.data))
    return y


def quantize(typ, x):
    x = np.ascontiguousarray(x, dtype=np.float32)
    rows, k = int(np.prod(x.shape[:-1])), x.shape[-1]
    out = np.empty(rows * _gguf.row_bytes(typ, k), dtype=np.uint8)
    _lib.check(_lib.load().b200_quantize(typ, x.ctypes.data, rows, k, out.ctypes.data))
    return out
