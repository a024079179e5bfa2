"""GGUF v3 container: a writer for synthetic checkpoints and an mmap reader.

Mirrors the container the reference reads (gguf/gguf.go:293-403): magic, version,
tensor and key/value counts, the KV table, the tensor table `(name, n_dims, dims[], type,
offset)`, then the data section aligned to `general.alignment` (default 32). Dims are in
ggml order: dims[0] is the row length and the quantised axis (gguf/gguf.go:23-27).

The C++ library has its own reader (csrc/gguf_reader.cpp); this one serves the Python
host side and the tests, which cross-check the two.
"""
import mmap
import struct

import numpy as np

MAGIC = b"GGUF"

# ggml tensor types (gguf/gguf.go:53-88) -> (elements per block, bytes per block)
F32, F16, Q4_0, Q4_1, Q5_0, Q5_1, Q8_0 = 0, 1, 2, 3, 6, 7, 8
Q4_K, Q5_K, Q6_K, IQ4_NL, BF16 = 12, 13, 14, 20, 30
BLOCK = {F32: (1, 4), F16: (1, 2), BF16: (1, 2), Q4_1: (32, 20), Q5_0: (32, 22), Q5_1: (32, 24), Q8_0: (32, 34),
         IQ4_NL: (32, 18), Q4_K: (256, 144), Q5_K: (256, 176), Q6_K: (256, 210)}
TYPE_NAME = {F32: "F32", F16: "F16", BF16: "BF16", Q4_1: "Q4_1", Q5_0: "Q5_0", Q5_1: "Q5_1", Q8_0: "Q8_0",
             IQ4_NL: "IQ4_NL", Q4_K: "Q4_K", Q5_K: "Q5_K", Q6_K: "Q6_K"}

# metadata value tags (gguf/gguf.go:501-518)
U8, I8, U16, I16, U32, I32, FLT32, BOOL, STR, ARR, U64, I64, FLT64 = range(13)
_SCALAR = {U8: "<B", I8: "<b", U16: "<H", I16: "<h", U32: "<I", I32: "<i", FLT32: "<f", BOOL: "<?", U64: "<Q", I64: "<q", FLT64: "<d"}


def row_bytes(typ, n):
    e, b = BLOCK[typ]
    if n % e:
        raise ValueError(f"{n} elements is not a whole number of {TYPE_NAME[typ]} blocks of {e}")
    return n // e * b


def tensor_bytes(typ, dims):
    n = 1
    for d in dims[1:]:
        n *= d
    return row_bytes(typ, dims[0]) * n


def _wstr(s):
    b = s.encode()
    return struct.pack("<Q", len(b)) + b


class Writer:
    """Collects metadata and tensors, then writes one GGUF v3 file."""

    def __init__(self, arch, alignment=32):
        self.kv = []
        self.tensors = []
        self.alignment = alignment
        self.add("general.architecture", STR, arch)
        self.add("general.alignment", U32, alignment)

    def add(self, key, tag, value, elem_tag=None):
        self.kv.append((key, tag, value, elem_tag))

    def add_tensor(self, name, typ, dims, data):
        data = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
        want = tensor_bytes(typ, dims)
        if data.size != want:
            raise ValueError(f"{name}: {data.size} bytes for {TYPE_NAME[typ]} {list(dims)}, want {want}")
        self.tensors.append((name, typ, tuple(int(d) for d in dims), data))

    def _value(self, tag, v, elem_tag):
        if tag == STR:
            return _wstr(v)
        if tag == ARR:
            out = struct.pack("<IQ", elem_tag, len(v))
            for x in v:
                out += self._value(elem_tag, x, None)
            return out
        return struct.pack(_SCALAR[tag], v)

    def write(self, path):
        head = MAGIC + struct.pack("<IQQ", 3, len(self.tensors), len(self.kv))
        for key, tag, v, et in self.kv:
            head += _wstr(key) + struct.pack("<I", tag) + self._value(tag, v, et)
        off, offs = 0, []
        for _, typ, dims, data in self.tensors:
            offs.append(off)
            off += (data.size + self.alignment - 1) // self.alignment * self.alignment
        for (name, typ, dims, _), o in zip(self.tensors, offs):
            head += _wstr(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims)
            head += struct.pack("<IQ", typ, o)
        pad = (-len(head)) % self.alignment
        with open(path, "wb") as f:
            f.write(head + b"\0" * pad)
            for _, _, _, data in self.tensors:
                f.write(data.tobytes())
                f.write(b"\0" * ((-data.size) % self.alignment))


def write_split(path_stem, arch, metadata, tensors, n_shards, alignment=32):
    """Writes a checkpoint as `n_shards` files `<stem>-0000i-of-0000n.gguf` in llama.cpp's split convention
    (gguf/gguf.go:726-733): every shard a whole GGUF with its own tensor table, the first carrying the model's
    metadata, each carrying split.no / split.count / split.tensors.count. Returns the paths."""
    names = list(tensors)
    per = (len(names) + n_shards - 1) // n_shards
    paths = []
    for i in range(n_shards):
        w = Writer(arch, alignment)
        if i == 0:
            for row in metadata:
                w.add(*row)
        w.add("split.no", U16, i)
        w.add("split.count", U16, n_shards)
        w.add("split.tensors.count", I32, len(names))
        for name in names[i * per:(i + 1) * per]:
            typ, dims, data = tensors[name]
            w.add_tensor(name, typ, dims, data)
        paths.append(f"{path_stem}-{i + 1:05d}-of-{n_shards:05d}.gguf")
        w.write(paths[-1])
    return paths


class Reader:
    """mmap view of one GGUF file: `.kv` dict and `.tensors` {name: (type, dims, uint8 view)}."""

    def __init__(self, path):
        self._f = open(path, "rb")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        b, self._o = self._mm, 0
        if b[:4] != MAGIC:
            raise ValueError(f"{path}: not a GGUF file")
        self._o = 4
        self.version, nt, nkv = self._unpack("<IQQ")
        if self.version not in (2, 3):
            raise ValueError(f"{path}: GGUF version {self.version} is not 2 or 3")
        self.kv = {}
        for _ in range(nkv):
            key = self._str()
            (tag,) = self._unpack("<I")
            self.kv[key] = self._value(tag)
        infos = []
        for _ in range(nt):
            name = self._str()
            (nd,) = self._unpack("<I")
            dims = self._unpack("<" + "Q" * nd)
            typ, off = self._unpack("<IQ")
            infos.append((name, typ, dims, off))
        align = int(self.kv.get("general.alignment", 32))
        base = (self._o + align - 1) // align * align
        whole = np.frombuffer(self._mm, dtype=np.uint8)
        self.tensors = {}
        for name, typ, dims, off in infos:
            if typ not in BLOCK:
                raise ValueError(f"{name}: unsupported ggml type {typ}")
            nb = tensor_bytes(typ, dims)
            if base + off + nb > whole.size:
                raise ValueError(f"{name}: data runs past the end of the file")
            self.tensors[name] = (typ, tuple(dims), whole[base + off: base + off + nb])

    def _unpack(self, fmt):
        v = struct.unpack_from(fmt, self._mm, self._o)
        self._o += struct.calcsize(fmt)
        return v

    def _str(self):
        (n,) = self._unpack("<Q")
        s = self._mm[self._o:self._o + n].decode()
        self._o += n
        return s

    def _value(self, tag):
        if tag == STR:
            return self._str()
        if tag == ARR:
            et, n = self._unpack("<IQ")
            return [self._value(et) for _ in range(n)]
        return self._unpack(_SCALAR[tag])[0]

    @property
    def arch(self):
        return self.kv.get("general.architecture", "")


def model_config(kv, tensors):
    """The hyper-parameters the graph needs, read the way the reference reads them
    (llm/model.go:66-96, 375-407, 441-468). Returns a dict of plain ints/floats."""
    arch = kv.get("general.architecture", "")
    if not arch:
        raise ValueError("checkpoint states no general.architecture")
    g = lambda k, d=0: kv.get(f"{arch}.{k}", d)
    n_layer = int(g("block_count"))
    draft = int(g("nextn_predict_layers", 0))
    cfg = dict(
        n_layer=n_layer - draft, n_embd=int(g("embedding_length")), vocab=int(tensors["token_embd.weight"][1][1]),
        n_head=int(g("attention.head_count")), n_head_kv=int(g("attention.head_count_kv")),
        head_dim=int(g("attention.key_length")), rope_dims=int(g("rope.dimension_count")),
        rope_base=float(g("rope.freq_base", 10000.0)), eps=float(g("attention.layer_norm_rms_epsilon", 1e-6)),
        n_expert=int(g("expert_count")), n_expert_used=int(g("expert_used_count")),
        ffn_expert=int(g("expert_feed_forward_length")),
        ffn_shared=int(g("expert_shared_feed_forward_length", g("expert_feed_forward_length"))),
        dn_head_dim=int(g("ssm.state_size")), dn_heads_k=int(g("ssm.group_count")), dn_heads_v=int(g("ssm.time_step_rank")),
        dn_conv=int(g("ssm.conv_kernel")), has_draft=1 if draft else 0)
    return cfg
