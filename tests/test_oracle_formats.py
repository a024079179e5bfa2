"""Pins the oracle's block formats, quantiser and fp16 rounding against the reference's
committed known-answer fixtures (copies under tests/golden/, made by make_fixtures.py)."""
import os
import struct

import numpy as np
import pytest

from conftest import GOLDEN


def _dequant_records(path):
    b = open(path, "rb").read()
    o, out = 0, []
    while o < len(b):
        t, n, nb = struct.unpack_from("<IIQ", b, o); o += 16
        out.append((t, n, b[o:o + nb])); o += nb
    return out


def _quant_records(path):
    b = open(path, "rb").read()
    o, out = 0, []
    while o < len(b):
        t, r, k, im = struct.unpack_from("<IIII", b, o); o += 16
        out.append((t, r, k, np.frombuffer(b[o:o + 4 * r * k], dtype=np.float32).reshape(r, k))); o += 4 * r * k
    return out


def test_f32_to_f16_matches_fixture(orc):
    # safetensors/testdata/f32_to_f16.txt: round-to-nearest-even including subnormals
    n = 0
    for line in open(os.path.join(GOLDEN, "f32_to_f16.txt")):
        if line.startswith("#") or not line.strip():
            continue
        a, b = line.split()
        f = np.array([int(a, 16)], dtype=np.uint32).view(np.float32)[0]
        assert orc.lib().orc_f32_to_f16(float(f)) == int(b, 16), a
        n += 1
    assert n > 10000


def test_f16_to_f32_every_half(orc):
    h = np.arange(65536, dtype=np.uint16)
    ref = h.view(np.float16).astype(np.float32)
    got = np.array([orc.lib().orc_f16_to_f32(int(x)) for x in h], dtype=np.float32)
    ok = (got.view(np.uint32) == ref.view(np.uint32)) | (np.isnan(got) & np.isnan(ref))
    assert ok.all()


def test_dequant_matches_ggml_fixture_bit_exact(orc):
    # gguf/dequant_test.go:40-98 TestDequantMatchesGGML: all 11 formats, every float exact
    rin = _dequant_records(os.path.join(GOLDEN, "dequant_in.bin"))
    rref = _dequant_records(os.path.join(GOLDEN, "dequant_ref.bin"))
    assert [r[0] for r in rin] == [12, 13, 7, 8, 20, 0, 1, 30, 3, 6, 14]
    for (t, n, payload), (t2, n2, ref) in zip(rin, rref):
        assert (t, n) == (t2, n2)
        got = orc.dequantize(t, payload, n)
        assert np.array_equal(got.view(np.uint32), np.frombuffer(ref, dtype=np.uint32)), f"type {t}"


def test_dequant_refuses_partial_blocks(orc):
    with pytest.raises(ValueError):
        orc.dequantize(12, bytes(144), 100)
    with pytest.raises(ValueError):
        orc.dequantize(99, bytes(144), 256)


def test_quantiser_round_trip_matches_ggml_fixture(orc):
    # llm/quantref_test.go:27-31: equality after rounding both sides to fp16 is the reference's
    # bar; the oracle meets the stronger one (identical f32).
    rin = _quant_records(os.path.join(GOLDEN, "quant_subset_in.bin"))
    rref = _quant_records(os.path.join(GOLDEN, "quant_subset_ref.bin"))
    assert len(rin) == 4
    for (t, r, k, x), (_, _, _, ref) in zip(rin, rref):
        d = orc.dequantize(t, orc.quantize(t, x), r * k).reshape(r, k)
        assert np.array_equal(d.astype(np.float16), ref.astype(np.float16)), (t, k)
        assert np.array_equal(d.view(np.uint32), ref.view(np.uint32)), (t, k)


@pytest.mark.parametrize("typ", [8, 12, 13, 14])
def test_quantise_dequantise_error_is_small(orc, typ):
    rng = np.random.default_rng(3)
    x = (0.02 * rng.standard_normal((8, 1024))).astype(np.float32)
    d = orc.dequantize(typ, orc.quantize(typ, x), x.size).reshape(x.shape)
    rel = np.sqrt(np.mean((d - x) ** 2)) / np.sqrt(np.mean(x ** 2))
    assert rel < {8: 0.01, 12: 0.09, 13: 0.05, 14: 0.025}[typ]


def test_scale_min_pack_round_trip(orc):
    # llm/bank_q4_test.go TestQ4KRecordPackings: the 12-byte packing survives a decode
    rng = np.random.default_rng(5)
    x = (rng.standard_normal((4, 256)) * np.linspace(0.01, 3, 8).repeat(32)).astype(np.float32)
    q = orc.quantize(12, x)
    d = orc.dequantize(12, q, x.size).reshape(x.shape)
    assert np.abs(d - x).max() < 0.25 * np.abs(x).max()


def test_argmax_ties_to_lowest_id(orc):
    # llm/sample.go:359-367
    assert orc.argmax(np.array([1, 3, 3, 2], dtype=np.float32)) == 1
    assert orc.argmax(np.array([-np.inf, -np.inf], dtype=np.float32)) == 0


def test_fp16_weight_mode_rounds_only_the_named_matrices(orc, tiny_path):
    """The oracle's many-row arithmetic: dequantised weights rounded to fp16 (shaders/llm_gemm.comp MODE 2).
    With no bit set the result is the device-like one; the head bit alone changes only what the head does."""
    import modelgen
    om, cfg, _ = modelgen.oracle_model(tiny_path)
    ids = np.random.default_rng(2).integers(0, cfg["vocab"], 3).astype(np.int32)
    base, tb = om.seq().extend(ids, trace=("hidden",))
    same, _ = om.seq().extend(ids, numerics=orc.DEVICE_LIKE)
    assert np.array_equal(base, same)
    head, th = om.seq().extend(ids, numerics=orc.DEVICE_LIKE | orc.W16_HEAD, trace=("hidden",))
    assert np.array_equal(tb["hidden"], th["hidden"]) and not np.array_equal(base, head)
    for bit in range(8, 19):     # every named matrix is wired: its bit alone changes the result
        one, _ = om.seq().extend(ids, numerics=orc.DEVICE_LIKE | (1 << bit))
        assert not np.array_equal(one, base), f"bit {bit} has no effect"
        assert np.abs(one - base).max() < 3e-3 * np.abs(base).max()
    allw, ta = om.seq().extend(ids, numerics=orc.DEVICE_LIKE | orc.W16_ALL, trace=("hidden",))
    assert not np.array_equal(tb["hidden"], ta["hidden"])
    scale = np.abs(base).max()
    assert np.abs(head - base).max() < 2e-3 * scale and np.abs(allw - base).max() < 1e-2 * scale


def test_tensor_core_weights_are_the_rounded_value_or_a_neighbour(orc):
    """The fp16 weights of the many-row kernels (hi + lo factor pairs) against the reference's single rounding of
    the f32 value (shaders/llm_moe_gemm.comp:260-261): never further than one fp16 ulp, mostly identical."""
    rng = np.random.default_rng(9)
    for typ in (12, 13, 14, 8):
        q = orc.quantize(typ, (0.02 * rng.standard_normal((64, 1024))).astype(np.float32))
        exact = orc.dequantize(typ, q, 64 * 1024)
        once = exact.astype(np.float16)
        got = orc.dequantize_w16(typ, q, 64 * 1024)
        assert np.array_equal(got, got.astype(np.float16).astype(np.float32))      # fp16 values
        steps = np.abs(got.astype(np.float16).view(np.int16).astype(np.int32) - once.view(np.int16).astype(np.int32))
        steps[got == once.astype(np.float32)] = 0                                     # +0 against -0
        assert steps.max() <= 2, (typ, steps.max())
        assert (steps > 1).mean() < 1e-4 and (steps == 0).mean() > 0.8, (typ, (steps == 0).mean())
        if typ in (14, 8):
            assert steps.max() == 0                                                   # one factor: fp16(d * sc * q) is the single rounding
