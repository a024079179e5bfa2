"""The allocation-free projection entry point against the ordinary one.

b200_qgemv_static() exists for hosts that cannot call cudaMalloc at the moment they need a
projection: a latency-critical thread that must not block on the allocator's lock, or a process
whose device memory was budgeted up front. It takes device pointers and stages the activations
in a fixed device array inside the library. This file is named so that pytest collects it last:
if it fails, every other test has already run.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _static_qgemv(pkg, torch, typ, q, rows, k, x, check_memory=False):
    w = torch.from_numpy(np.ascontiguousarray(q)).cuda()
    xd = torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)).cuda()
    yd = torch.empty((x.shape[0], rows), dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    st = pkg.lib.load().b200_qgemv_static(typ, C.c_void_p(w.data_ptr()), rows, k, C.c_void_p(xd.data_ptr()), x.shape[0], C.c_void_p(yd.data_ptr()))
    free1, _ = torch.cuda.mem_get_info()
    pkg.lib.check(st)
    if check_memory:
        # the property the entry point exists for: the device's free memory is what it was
        assert free1 == free0, (free0, free1)
    return yd.cpu().numpy()


def test_static_scratch_projection_matches_the_allocating_one(pkg, orc):
    torch = pytest.importorskip("torch")
    rng = np.random.default_rng(21)
    # the first call on a device looks up the arrays' addresses (and loads the kernel): memory is compared from the second on
    warm = orc.quantize(12, (0.02 * rng.standard_normal((16, 256))).astype(np.float32))
    _static_qgemv(pkg, torch, 12, warm, 16, 256, rng.standard_normal((1, 256)).astype(np.float32))
    # calls in a row on the shared staging array: later ones are smaller, so stale contents of an earlier
    # one would show if a call read more than it wrote. The last two sit at the documented limits:
    # 8 rows of 7680 (Q4_K) and one row of 16384.
    for typ, rows, k, m in ((12, 512, 2048, 8), (13, 256, 1024, 3), (12, 32, 7680, 8), (12, 16, 16384, 1), (13, 16, 7168, 8)):
        q = orc.quantize(typ, (0.02 * rng.standard_normal((rows, k))).astype(np.float32))
        x = rng.standard_normal((m, k)).astype(np.float32)
        want = pkg.qgemv(typ, q, rows, k, x)
        got = _static_qgemv(pkg, torch, typ, q, rows, k, x, check_memory=True)
        assert np.abs(got - want).max() <= 2e-5 * np.abs(want).max()
        assert np.array_equal(got, want)      # same kernel, same staged values: identical in practice


def test_static_scratch_projection_refuses_what_does_not_fit(pkg):
    torch = pytest.importorskip("torch")
    L = pkg.lib.load()
    buf = torch.zeros(1 << 20, dtype=torch.uint8, device="cuda")
    p = C.c_void_p(buf.data_ptr())
    assert L.b200_qgemv_static(12, p, 16, 256, p, 9, p) == pkg.lib.ECAPACITY        # more than 8 rows
    assert L.b200_qgemv_static(12, p, 16, 32768, p, 1, p) == pkg.lib.ECAPACITY      # row longer than the array
    # inside the array but beyond the kernel's shared memory: refused with the joint limit spelled out
    assert L.b200_qgemv_static(12, p, 16, 8192, p, 8, p) == pkg.lib.ECAPACITY
    msg = L.b200_last_error()
    assert b"8 rows of 8192" in msg and b"at most 7 rows fit" in msg, msg
    assert L.b200_qgemv_static(13, p, 16, 16384, p, 1, p) == pkg.lib.ECAPACITY      # Q5_K: one row stops at 16128
    assert b"no row fits" in L.b200_last_error()
    assert L.b200_qgemv_static(14, p, 16, 256, p, 1, p) == pkg.lib.EINVAL           # Q6_K needs a re-laid copy
    assert b"Q4_K" in L.b200_last_error()
