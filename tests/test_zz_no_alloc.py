"""The allocation-free projection entry point against the ordinary one.

b200_qgemv_static() exists for hosts that cannot call cudaMalloc when they need a projection:
code running inside a stream capture, a latency-critical thread that must not block on the
allocator's lock, or a process whose device memory was budgeted up front. It takes device
pointers and stages the activations in a fixed device array inside the library. This file is
named so that pytest collects it last: if it fails, every other test has already run.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _static_qgemv(pkg, torch, typ, q, rows, k, x):
    w = torch.from_numpy(np.ascontiguousarray(q)).cuda()
    xd = torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)).cuda()
    yd = torch.empty((x.shape[0], rows), dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    st = pkg.lib.load().b200_qgemv_static(typ, C.c_void_p(w.data_ptr()), rows, k, C.c_void_p(xd.data_ptr()), x.shape[0], C.c_void_p(yd.data_ptr()))
    pkg.lib.check(st)
    return yd.cpu().numpy()


def test_static_scratch_projection_matches_the_allocating_one(pkg, orc):
    torch = pytest.importorskip("torch")
    rng = np.random.default_rng(21)
    # two calls in a row on the shared staging array: the second is smaller, so stale contents
    # of the first would show if the call read more than it wrote
    for typ, rows, k, m in ((12, 512, 2048, 8), (13, 256, 1024, 3)):
        q = orc.quantize(typ, (0.02 * rng.standard_normal((rows, k))).astype(np.float32))
        x = rng.standard_normal((m, k)).astype(np.float32)
        want = pkg.qgemv(typ, q, rows, k, x)
        got = _static_qgemv(pkg, torch, typ, q, rows, k, x)
        assert np.abs(got - want).max() <= 2e-5 * np.abs(want).max()
        assert np.array_equal(got, want)      # same kernel, same staged values: identical in practice


def test_static_scratch_projection_refuses_what_does_not_fit(pkg):
    torch = pytest.importorskip("torch")
    L = pkg.lib.load()
    buf = torch.zeros(1 << 20, dtype=torch.uint8, device="cuda")
    p = C.c_void_p(buf.data_ptr())
    assert L.b200_qgemv_static(12, p, 16, 256, p, 9, p) == pkg.lib.ECAPACITY        # more than 8 rows
    assert L.b200_qgemv_static(12, p, 16, 32768, p, 1, p) == pkg.lib.ECAPACITY      # row longer than the array
    assert L.b200_qgemv_static(14, p, 16, 256, p, 1, p) == pkg.lib.EINVAL           # Q6_K needs a re-laid copy
    assert b"16384" in L.b200_last_error() or b"Q4_K" in L.b200_last_error()
