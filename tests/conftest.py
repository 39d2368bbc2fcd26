import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 GPU (the CUDA path through the C ABI)")


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def load_golden(name):
    return dict(np.load(os.path.join(GOLDEN, name)))


def coo_to_csr(g):
    import scipy.sparse as sp
    shape = tuple(int(x) for x in g["shape"])
    # coo -> csr keeps explicitly stored zeros, like the matrix the fixture was made from
    return sp.coo_matrix((g["coo_data"], (g["coo_row"], g["coo_col"])), shape=shape).tocsr()


def rel_err(got, ref):
    """The reference tests' metric: max|C - C_ref| / max|C_ref| (tests/test_all_features.py:43-48)."""
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    return float(np.abs(got - ref).max() / max(np.abs(ref).max(), 1e-30))
