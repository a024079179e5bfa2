"""B200-native token loop of a hybrid gated-DeltaNet / gated-GQA / MoE language model
stored as GGUF K-quants: hand-written CUDA for sm_100a behind a C ABI, plus the Python
mirror of the reference's `llm.Graph` interface used by the tests and the benchmark."""
from . import config, ep, gguf, lib, spec  # noqa: F401
from .graph import Graph, Model, dequantize, qgemm, qgemv, quantize  # noqa: F401
