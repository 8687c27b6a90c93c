import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    # GPU tests are skipped, not failed, where no device is visible and -m gpu was not asked for.
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


@pytest.fixture(scope="session")
def golden():
    def load(name):
        with np.load(os.path.join(GOLDEN, name)) as f:
            return {k: f[k] for k in f.files}
    return load


# ---- helpers shared by the GPU tests -------------------------------------------------------------

def to_dev(a, dtype=None):
    """numpy -> torch CUDA tensor; dtype "bf16" converts (the values must already be bf16-exact)."""
    import torch
    if a is None:
        return None
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    if dtype == "bf16":
        t = t.to(torch.bfloat16)
    return t


def to_np(t):
    import torch
    return t.detach().to(torch.float32).cpu().numpy()


def fp32_tol_err(got, ref):
    """max |got - ref| / (1 + |ref|): the fp32 parity gate is <= 1e-4."""
    return float(np.max(np.abs(got.astype(np.float64) - ref.astype(np.float64)) / (1.0 + np.abs(ref.astype(np.float64)))))


def rel_l2(got, ref):
    """relative L2 error: the bf16-input gate is <= 2e-2 against the fp32 oracle."""
    g, r = got.astype(np.float64), ref.astype(np.float64)
    return float(np.linalg.norm(g - r) / max(np.linalg.norm(r), 1e-30))


FP32_TOL = 1e-4
BF16_TOL = 2e-2
