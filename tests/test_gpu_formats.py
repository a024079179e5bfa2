"""GPU parity of the block formats, the device quantiser and the fused K-quant projection
kernel against the oracle and the reference's golden fixtures. Everything goes through the C ABI."""
import os
import struct

import numpy as np
import pytest

from conftest import GOLDEN
from test_oracle_formats import _dequant_records, _quant_records

pytestmark = pytest.mark.gpu

DEVICE_TYPES = {0, 1, 30, 8, 12, 13, 14}


def test_device_dequant_matches_ggml_fixture_bit_exact(pkg):
    # gguf/dequant_test.go:40-98, for the formats the device layout carries
    rin = _dequant_records(os.path.join(GOLDEN, "dequant_in.bin"))
    rref = _dequant_records(os.path.join(GOLDEN, "dequant_ref.bin"))
    seen = 0
    for (t, n, payload), (_, _, ref) in zip(rin, rref):
        if t not in DEVICE_TYPES:
            continue
        got = pkg.dequantize(t, payload, n)
        assert np.array_equal(got.view(np.uint32), np.frombuffer(ref, dtype=np.uint32)), f"type {t}"
        seen += 1
    assert seen == 7


@pytest.mark.parametrize("typ", [8, 12, 13, 14])
def test_device_quantiser_is_the_oracles(pkg, orc, typ):
    rng = np.random.default_rng(7)
    x = (0.02 * rng.standard_normal((64, 2048))).astype(np.float32)
    x[3, :256] = 0.0          # an all-zero super-block
    x[5, 256:288] = 0.5       # a constant group
    assert np.array_equal(pkg.quantize(typ, x), orc.quantize(typ, x))


def test_device_quantiser_matches_ggml_fixture(pkg, orc):
    # llm/quantref_test.go: round trip equals ggml's after fp16 rounding (here: exactly)
    rin = _quant_records(os.path.join(GOLDEN, "quant_subset_in.bin"))
    rref = _quant_records(os.path.join(GOLDEN, "quant_subset_ref.bin"))
    for (t, r, k, x), (_, _, _, ref) in zip(rin, rref):
        d = pkg.dequantize(t, pkg.quantize(t, x), r * k).reshape(r, k)
        assert np.array_equal(d.view(np.uint32), ref.view(np.uint32)), (t, k)


@pytest.mark.parametrize("typ", [12, 13, 14])
@pytest.mark.parametrize("rows,k,m", [(16, 256, 1), (64, 512, 1), (48, 1024, 3), (4096, 1024, 1), (2048, 2048, 8), (2048, 4096, 2),
                                      (512, 2048, 11), (40, 768, 1)])
def test_qgemv_matches_oracle_matvec(pkg, orc, typ, rows, k, m):
    rng = np.random.default_rng(rows * 31 + k + m)
    w = (0.02 * rng.standard_normal((rows, k))).astype(np.float32)
    q = orc.quantize(typ, w)
    x = rng.standard_normal((m, k)).astype(np.float32)
    x16 = x.astype(np.float16).astype(np.float32)   # the kernel stages activations as fp16
    got = pkg.qgemv(typ, q, rows, k, x)
    want = np.stack([orc.matvec(typ, q, rows, k, x16[i]) for i in range(m)])
    scale = np.abs(want).max()
    # f32 accumulation in another order; Q6_K additionally rounds sc*(q-32) above 2048 to fp16
    tol = 2e-5 if typ != 14 else 2e-4
    assert np.abs(got - want).max() <= tol * scale, (np.abs(got - want).max(), scale)


def test_qgemv_columns_are_independent(pkg, orc):
    # a batched pass equals each row stepped alone (llm/graph_batch_test.go:13-33), bit for bit
    rng = np.random.default_rng(11)
    rows, k = 256, 2048
    q = orc.quantize(12, (0.02 * rng.standard_normal((rows, k))).astype(np.float32))
    x = rng.standard_normal((8, k)).astype(np.float32)
    both = pkg.qgemv(12, q, rows, k, x)
    for i in (0, 3, 7):
        alone = pkg.qgemv(12, q, rows, k, x[i:i + 1])
        assert np.array_equal(both[i].view(np.uint32), alone[0].view(np.uint32))


def test_refusals(pkg):
    with pytest.raises(pkg.lib.B200Error):
        pkg.dequantize(12, bytes(144), 100)
    with pytest.raises(pkg.lib.B200Error):
        pkg.qgemv(8, bytes(34 * 8), 1, 256, np.zeros(256, dtype=np.float32))   # Q8_0 has no fused projection
