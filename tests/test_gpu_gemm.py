"""GPU parity of the tensor-core (tcgen05 / TMEM) many-row projection against a CPU restatement of the
reference's prefill GEMM arithmetic: K-quant weights dequantised in f32, rounded to fp16, multiplied
with fp16 activations, accumulated in f32 (shaders/llm_gemm.comp MODE 2)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

# The kernel forms each weight in fp16 arithmetic (within about one fp16 ulp of the f32 value rounded
# once) and sums in a different order: 5e-4 of the output scale.
TOL = 5e-4


def _want(orc, typ, q, rows, k, x):
    w16 = orc.dequantize(typ, q, rows * k).reshape(rows, k).astype(np.float16).astype(np.float64)
    x16 = x.astype(np.float16).astype(np.float64)
    return (x16 @ w16.T).astype(np.float32)


@pytest.mark.parametrize("typ", [12, 13, 14])
@pytest.mark.parametrize("rows,k,m,tile", [(128, 256, 64, 64), (256, 512, 100, 64), (384, 2048, 300, 128), (200, 768, 33, 64),
                                           (1024, 2048, 520, 256), (128, 4096, 17, 128)])
def test_qgemm_matches_fp16_weight_product(pkg, orc, typ, rows, k, m, tile):
    rng = np.random.default_rng(rows * 7 + k + m)
    w = (0.02 * rng.standard_normal((rows, k))).astype(np.float32)
    q = orc.quantize(typ, w)
    x = rng.standard_normal((m, k)).astype(np.float32)
    got = pkg.qgemm(typ, q, rows, k, x, tile)
    want = _want(orc, typ, q, rows, k, x)
    scale = np.abs(want).max()
    assert np.abs(got - want).max() <= TOL * scale, (np.abs(got - want).max(), scale)


@pytest.mark.parametrize("typ", [12, 13, 14, 8])
def test_qgemm_multiplies_the_weights_the_oracle_names(pkg, orc, typ):
    """The oracle's many-row mode states the fp16 weights bit for bit (hi + lo factor pairs): against a product
    over exactly those weights only the summation order differs."""
    rng = np.random.default_rng(31 + typ)
    rows, k, m = 256, 2048, 96
    q = orc.quantize(typ, (0.02 * rng.standard_normal((rows, k))).astype(np.float32))
    x = rng.standard_normal((m, k)).astype(np.float32)
    got = pkg.qgemm(typ, q, rows, k, x, 64)
    w = orc.dequantize_w16(typ, q, rows * k).reshape(rows, k).astype(np.float64)
    want = (x.astype(np.float16).astype(np.float64) @ w.T).astype(np.float32)
    assert np.abs(got - want).max() <= 1e-5 * np.abs(want).max(), np.abs(got - want).max()   # tensor-core accumulation is not exactly f32


@pytest.mark.parametrize("rows,k,m", [(512, 2048, 300), (128, 256, 5), (96, 1024, 70)])
def test_qgemm_q8_0_router_weights(pkg, orc, rows, k, m):
    # the router's weight type, 64-row tiles only (many-row passes compute the router logits this way)
    rng = np.random.default_rng(rows + k + m)
    q = orc.quantize(8, (0.02 * rng.standard_normal((rows, k))).astype(np.float32))
    x = rng.standard_normal((m, k)).astype(np.float32)
    got = pkg.qgemm(8, q, rows, k, x, 64)
    want = _want(orc, 8, q, rows, k, x)
    assert np.abs(got - want).max() <= TOL * np.abs(want).max()


def test_qgemm_agrees_with_the_few_row_kernel(pkg, orc):
    # the two projection kernels differ only by the fp16 rounding of the weights
    rng = np.random.default_rng(5)
    rows, k, m = 256, 2048, 8
    q = orc.quantize(12, (0.02 * rng.standard_normal((rows, k))).astype(np.float32))
    x = rng.standard_normal((m, k)).astype(np.float32)
    a, b = pkg.qgemm(12, q, rows, k, x, 64), pkg.qgemv(12, q, rows, k, x)
    assert np.abs(a - b).max() <= 2e-3 * np.abs(b).max()


def test_qgemm_refusals(pkg, orc):
    # refused on the host before anything is launched
    q = orc.quantize(12, np.zeros((128, 256), dtype=np.float32))
    x = np.zeros((4, 256), dtype=np.float32)
    with pytest.raises(pkg.lib.B200Error):
        pkg.qgemm(12, q, 128, 256, x, 96)          # tiles are 64, 128 or 256 rows
    with pytest.raises(pkg.lib.B200Error):
        pkg.qgemm(8, orc.quantize(8, np.zeros((128, 256), dtype=np.float32)), 128, 256, x, 128)   # Q8_0: 64-row tiles only
    with pytest.raises(pkg.lib.B200Error):
        pkg.qgemm(0, np.zeros(128 * 256 * 4, dtype=np.uint8), 128, 256, x, 64)   # F32 weights have no kernel
