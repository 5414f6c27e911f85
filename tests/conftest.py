import json
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def oracle():
    import oracle as orc
    if not os.path.exists(orc.ORACLE_LIB):
        orc.build(ref=False)
    return orc.Oracle()


@pytest.fixture(scope="session")
def reference():
    """The reference's own sources compiled in place; only where that build exists."""
    import oracle as orc
    if not orc.Reference.available():
        pytest.skip("oracle/_ref not built on this machine (needs the reference tree)")
    return orc.Reference()


@pytest.fixture(scope="session")
def kats():
    with open(os.path.join(GOLDEN, "kats.json")) as f:
        return json.load(f)


@pytest.fixture(scope="session")
def cuda_device():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda", 0)


def random_csr(rng, rows, cols, max_nnz, bits, policy=1, empty_rows=True):
    """Small random quantized-CSR input (float values near a per-gene affine grid)."""
    counts = rng.integers(0 if empty_rows else 1, max_nnz + 1, size=rows)
    counts = np.minimum(counts, cols)
    row_ptr = np.zeros(rows + 1, dtype=np.int64)
    np.cumsum(counts, out=row_ptr[1:])
    col_idx = np.concatenate([np.sort(rng.choice(cols, size=int(c), replace=False)) for c in counts]
                             + [np.zeros(0, dtype=np.int64)]).astype(np.int32)
    scales = rng.uniform(0.01, 0.5, size=cols).astype(np.float32)
    scales[rng.integers(0, cols)] = 0.0  # the scale == 0 rule
    n_off = cols if policy == 1 else rows
    offsets = rng.uniform(-1.0, 1.0, size=n_off).astype(np.float32)
    values = rng.uniform(-2.0, 40.0, size=len(col_idx)).astype(np.float32)
    return dict(rows=rows, cols=cols, bits=bits, policy=policy, row_ptr=row_ptr, col_idx=col_idx, scales=scales,
                offsets=offsets, values=values)
