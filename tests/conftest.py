import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(autouse=True)
def _seed():
    torch.manual_seed(0)


def load_golden(name):
    """Golden .npz -> dict of torch tensors (bf16 restored from its bit pattern)."""
    out = {}
    with np.load(os.path.join(GOLDEN, name + ".npz")) as z:
        for key in z.files:
            a = z[key]
            if key.endswith("__bf16"):
                out[key[:-6]] = torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)
            elif a.ndim == 0 and a.dtype.kind in "US":
                out[key] = str(a)
            else:
                out[key] = torch.from_numpy(a.copy())
    return out


def rel_l2(a, b):
    a, b = a.float(), b.float()
    return float((a - b).norm() / b.norm().clamp(min=1e-30))
