"""Test configuration: registers the `gpu` marker and puts the package and the oracle on sys.path.

`-m "not gpu"` covers the oracle against the golden vectors, the host-side front end and the
symbol table of the C-ABI library; `-m gpu` holds the parity tests, which call the CUDA kernels
through the C ABI and compare with the oracle.
"""
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
PKG = ROOT / "tilelang-tpu_b200"
for p in (str(PKG), str(ROOT)):
    if p not in sys.path:
        sys.path.insert(0, p)

GOLDEN = Path(__file__).resolve().parent / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a)")


def load_golden(name: str, dtypes: dict | None = None) -> dict:
    """Load tests/golden/<name>.npz; `dtypes` maps array name -> torch dtype for arrays stored as
    raw bit patterns (uint16 for 16-bit floats, uint8 for e4m3)."""
    dtypes = dtypes or {}
    out = {}
    with np.load(GOLDEN / f"{name}.npz") as z:
        for k in z.files:
            a = z[k]
            if a.shape == ():
                out[k] = a.item()
                continue
            t = torch.from_numpy(a.copy())
            if k in dtypes:
                t = t.view(dtypes[k])
            out[k] = t
    return out


@pytest.fixture(scope="session")
def cuda_device():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    torch.cuda.set_device(0)
    return torch.device("cuda", 0)
