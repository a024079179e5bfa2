"""Seeded synthetic checkpoints for the tests: values drawn per the manifest's rules from
numpy's default_rng(seed) in manifest order, quantised by the oracle's quantiser
(uncalibrated arm), written as GGUF by the package's writer."""
import importlib
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "oracle"))
import orc  # noqa: E402

pkg = importlib.import_module("strix-halo-vulkan_b200")
gguf, config = pkg.gguf, pkg.config


def draw(rng, rule, n):
    kind, a, b = rule
    if kind == "normal":
        return (a + b * rng.standard_normal(n, dtype=np.float32)).astype(np.float32)
    if kind == "neg_exp_uniform":
        return (-np.exp(rng.uniform(a, b, n))).astype(np.float32)
    raise ValueError(kind)


def build_tensors(cfg, seed=0):
    """{name: (type, dims, uint8 array)} for every tensor of the manifest."""
    rng = np.random.default_rng(seed)
    out = {}
    for name, typ, dims, rule in config.manifest(cfg):
        n = int(np.prod(dims))
        x = draw(rng, rule, n).reshape(-1, dims[0])
        out[name] = (typ, tuple(dims), orc.quantize(typ, x))
    return out


def write_gguf(cfg, path, seed=0, arch="qwen3next"):
    tensors = build_tensors(cfg, seed)
    w = gguf.Writer(arch)
    for row in config.metadata(cfg, arch):
        w.add(*row)
    for name, (typ, dims, data) in tensors.items():
        w.add_tensor(name, typ, dims, data)
    w.write(path)
    return tensors


def cached_gguf(cfg, seed=0, tag=None):
    """Path of the checkpoint for (cfg, seed), generated once per machine under the temp dir."""
    import hashlib
    import tempfile
    key = hashlib.sha1(repr((sorted((k, str(v)) for k, v in cfg.items()), seed)).encode()).hexdigest()[:12]
    d = os.path.join(tempfile.gettempdir(), "b200_llm_models")
    os.makedirs(d, exist_ok=True)
    path = os.path.join(d, f"{tag or cfg['name']}-{key}.gguf")
    if not os.path.exists(path):
        write_gguf(cfg, path + ".tmp", seed)
        os.replace(path + ".tmp", path)
    return path


def oracle_model(path):
    r = gguf.Reader(path)
    cfg = gguf.model_config(r.kv, r.tensors)
    return orc.Model(cfg, r.tensors), cfg, r
