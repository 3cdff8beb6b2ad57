import json
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
GOLDEN = os.path.join(ROOT, "tests", "golden")

# tolerances of the reference's own kernel tests (tests/conftest.py:53-55 there): |err| <= 1e-5 * sum|w x| for FP32
# accumulation, 2^-8 relative for a BF16 output; the hard gate of this build is 2^-10 of sum|w x| against FP64
GEMV_REL = 1e-5
HARD_REL = 2.0 ** -10
BF16_REL = 2.0 ** -8


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def golden_vectors():
    with open(os.path.join(GOLDEN, "encoder_vectors.json")) as f:
        meta = json.load(f)
    return meta, np.load(os.path.join(GOLDEN, "encoder_vectors.npz"))


@pytest.fixture(scope="session")
def policy_table():
    with open(os.path.join(GOLDEN, "policy_table.json")) as f:
        return json.load(f)


def to_bf16_tensor(bits: np.ndarray):
    import torch
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16).copy()).view(torch.bfloat16)


def bits_of(t) -> np.ndarray:
    import torch
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)
