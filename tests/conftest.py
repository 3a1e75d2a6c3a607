import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); deselect with -m 'not gpu'")


def load_model(name):
    """Model tables of the reference fixture `name` ('3mer' / '5mer') as torch CPU tensors."""
    import torch
    z = np.load(os.path.join(GOLDEN, f"hmm_{name}.npz"))
    return {k: torch.from_numpy(np.asarray(z[k])) for k in z.files}


def load_signals(indices=None):
    """The 100 nanopore reads of the reference fixture (zero padded int8) as a `seqs` dict."""
    import torch
    z = np.load(os.path.join(GOLDEN, "signals.npz"))
    data, lens = z["data"], z["lens"]
    if indices is not None:
        data, lens = data[indices], lens[indices]
        data = data[:, :int(lens.max())]
    return {
        "data": torch.from_numpy(np.ascontiguousarray(data)),
        "lens": torch.from_numpy(np.ascontiguousarray(lens)),
        "maxlen": torch.tensor(data.shape[1], dtype=torch.int64),
        "num_instances": torch.tensor(data.shape[0], dtype=torch.int64),
    }


def load_expected(name):
    return np.load(os.path.join(GOLDEN, "expected.npz"))["expected_" + name]


def shortest_reads(n):
    z = np.load(os.path.join(GOLDEN, "signals.npz"))
    return np.sort(np.argsort(z["lens"], kind="stable")[:n])


def max_rel(a, b):
    """Largest relative error; entries where both sides hold the same infinity
    count as exact, a one-sided infinity or any NaN as infinite error."""
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    same_inf = np.isinf(a) & np.isinf(b) & (np.sign(a) == np.sign(b))
    with np.errstate(invalid="ignore"):
        err = np.abs(a - b) / np.maximum(np.abs(b), 1e-30)
    err = np.where(same_inf, 0.0, err)
    err = np.where(np.isnan(err), np.inf, err)
    return float(np.max(err)) if err.size else 0.0


@pytest.fixture(scope="session")
def native():
    """The loaded C-ABI library; GPU tests fail (not skip) when it is missing."""
    from parpy_b200 import _native
    return _native
