import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except Exception:
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def load_golden(name):
    """Golden fixture as a dict of numpy arrays; bf16 tensors (stored as int16 bit patterns) come back as torch bf16."""
    import torch
    d = dict(np.load(os.path.join(GOLDEN, name + ".npz")))
    out = {}
    for k, v in d.items():
        if k.endswith("__bf16"):
            out[k[:-6]] = torch.from_numpy(v.copy()).view(torch.bfloat16)
        else:
            out[k] = v
    return out


def to_np(x):
    """numpy fp32 view of a golden entry (torch bf16 or numpy)."""
    import torch
    if isinstance(x, torch.Tensor):
        return x.float().numpy()
    return x


@pytest.fixture(scope="session")
def oracle():
    from oracle import jetfire_oracle as O
    O.build_c_oracle()
    return O


@pytest.fixture(scope="session")
def NL():
    from jetfire_int8training_b200 import Nonlinear
    return Nonlinear
