import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    try:
        import torch
        have = torch.cuda.is_available()
    except Exception:
        have = False
    if have:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


# Tolerance north star: GEMV / attention / logits within 1e-3 relative and 1e-4 absolute in f32.
RTOL, ATOL = 1.0e-3, 1.0e-4


def assert_close(actual, expected, rtol=RTOL, atol=ATOL, what=""):
    a = np.asarray(actual, dtype=np.float64).ravel()
    e = np.asarray(expected, dtype=np.float64).ravel()
    assert a.shape == e.shape, f"{what}: shape {a.shape} vs {e.shape}"
    bad = ~(np.abs(a - e) <= atol + rtol * np.abs(e))
    if bad.any():
        i = int(np.argmax(np.abs(a - e) - (atol + rtol * np.abs(e))))
        raise AssertionError(f"{what}: {int(bad.sum())}/{a.size} outside rtol={rtol} atol={atol}; worst at {i}: "
                             f"got {a[i]!r}, expected {e[i]!r}")


def assert_bit_exact(actual, expected, what=""):
    a = np.ascontiguousarray(actual, dtype=np.float32).ravel().view(np.uint32)
    e = np.ascontiguousarray(expected, dtype=np.float32).ravel().view(np.uint32)
    assert a.shape == e.shape, f"{what}: shape {a.shape} vs {e.shape}"
    if not np.array_equal(a, e):
        i = int(np.argmax(a != e))
        raise AssertionError(f"{what}: {int((a != e).sum())}/{a.size} words differ; first at {i}: {a[i]:#010x} vs {e[i]:#010x}")


@pytest.fixture(scope="session")
def golden():
    return np.load(os.path.join(ROOT, "tests", "golden", "dequant_golden.npz"))
