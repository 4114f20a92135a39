import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "customize-block-sparse-attention-with-triton_b200")
for p in (PKG, ROOT):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 GPU (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def lib():
    """The built C-ABI library; building happens in-tree (cross-compiles without a GPU)."""
    sys.path.insert(0, PKG)
    import build as _build
    _build.build()
    from fa2_custom_mask import _lib
    return _lib.load()


@pytest.fixture(scope="session")
def golden():
    import numpy as np
    gd = os.path.join(ROOT, "tests", "golden")
    return {n: np.load(os.path.join(gd, n + ".npz")) for n in ("groups", "fwd", "reorder")}


def golden_cases(npz):
    return sorted({k.split("/")[0] for k in npz.files})
