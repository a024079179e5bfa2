"""Comparison helpers shared by the parity tests."""
import numpy as np

# Tolerances of the contract: hidden states and logits within max relative error 1e-2
# (denominator floored at 1e-3, the reference's own compare(): llm/hc_test.go:52-83);
# routing indices and greedy ids exact unless the top-k margin / logit gap is below 1e-3.
REL_TOL = 1e-2
NEAR_TIE = 1e-3


def compare(got, want):
    got = np.asarray(got, dtype=np.float64).ravel()
    want = np.asarray(want, dtype=np.float64).ravel()
    assert got.shape == want.shape, (got.shape, want.shape)
    assert np.isfinite(got).all(), "non-finite values"
    d = np.abs(got - want)
    big = np.abs(want) > 1e-3
    return dict(max_abs=float(d.max()), max_rel=float((d[big] / np.abs(want[big])).max()) if big.any() else 0.0,
                rms=float(np.sqrt((d ** 2).mean())), ref_max=float(np.abs(want).max()))


def logit_gap(logits):
    top2 = np.partition(np.asarray(logits, dtype=np.float64), -2)[-2:]
    return float(top2[1] - top2[0])


def assert_close(got, want, what, tol=REL_TOL):
    r = compare(got, want)
    assert r["max_rel"] <= tol, f"{what}: {r}"
    return r
