"""pytest configuration: the ``gpu`` marker, path set-up and shared helpers."""
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


def load_golden(name):
    """A golden fixture as a dict of torch tensors (numpy scalars stay python numbers)."""
    out = {}
    with np.load(os.path.join(GOLDEN, name + ".npz")) as z:
        for k in z.files:
            a = z[k]
            out[k] = a.item() if a.ndim == 0 else torch.from_numpy(a.copy())
    return out


def norm_max_err(a, b):
    """max|a-b| / max|b|: the per-tensor metric the fp32 bar (1e-5) is stated on."""
    a = a.double().cpu(); b = b.double().cpu()
    return ((a - b).abs().max() / b.abs().max().clamp_min(1e-30)).item()


def bf16_violations(a, b, rtol=2e-2, atol=1e-2):
    """Fraction of elements with |a-b| > atol + rtol|b| (the bf16 bar), and the normalised max error."""
    a = a.double().cpu(); b = b.double().cpu()
    bad = ((a - b).abs() > atol + rtol * b.abs()).double().mean().item()
    return bad, norm_max_err(a, b)
