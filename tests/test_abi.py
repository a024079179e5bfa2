"""The C-ABI library loads and exports every symbol include/b200_llm.h declares (no GPU needed)."""
import os
import re

from conftest import ROOT


def test_header_symbols_are_exported(pkg):
    hdr = open(os.path.join(ROOT, "include", "b200_llm.h")).read()
    declared = set(re.findall(r"\b(b200_[a-z0-9_]+)\s*\(", hdr))
    assert len(declared) >= 40
    L = pkg.lib.load()
    for name in sorted(declared):
        assert hasattr(L, name), f"{name} is declared but not exported"
    assert declared == set(pkg.lib.SYMBOLS), declared ^ set(pkg.lib.SYMBOLS)


def test_product_fails_loudly_without_a_gpu(pkg):
    import pytest
    import numpy as np
    L = pkg.lib.load()
    if L.b200_device_count() > 0:
        pytest.skip("a GPU is present")
    with pytest.raises(pkg.lib.B200Error, match="no CPU path"):
        pkg.qgemv(12, bytes(144 * 16), 16, 256, np.zeros(256, dtype=np.float32))
