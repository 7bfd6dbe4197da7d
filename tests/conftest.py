import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = Path(__file__).resolve().parent / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def load_golden(name: str) -> dict:
    """Golden fixtures as torch tensors; bf16-exact inputs (stored as their upper 16 bits) come back as fp32."""
    out = {}
    with np.load(GOLDEN / name) as z:
        for k in z.files:
            a = z[k]
            if a.dtype == np.uint16:
                a = (a.astype(np.uint32) << 16).view(np.float32)
            out[k] = torch.from_numpy(np.ascontiguousarray(a))
    return out


@pytest.fixture(scope="session")
def golden_attention():
    return load_golden("attention_ref.npz")


@pytest.fixture(scope="session")
def golden_indices():
    return load_golden("indices_ref.npz")


@pytest.fixture(scope="session")
def golden_csla():
    return load_golden("csla_ref.npz")


@pytest.fixture(scope="session")
def golden_scalekv():
    return load_golden("scalekv_ref.npz")


@pytest.fixture(scope="session")
def golden_prologue():
    return load_golden("prologue_ref.npz")
