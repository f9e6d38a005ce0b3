"""Shared pytest configuration: markers, import path, golden-vector loader."""

import json
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = ROOT / "tests" / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def load_golden(name: str) -> dict:
    """Load tests/golden/<name>.npz as a dict of float64 torch tensors."""
    with np.load(GOLDEN / f"{name}.npz") as z:
        out = {}
        for key in z.files:
            arr = z[key]
            if key == "input_digest":
                out[key] = bytes(arr).decode()
            elif arr.dtype.kind == "f":
                out[key] = torch.from_numpy(arr.astype(np.float64))
            else:
                out[key] = arr
        return out


def load_kat(stem: str) -> dict:
    return json.loads((GOLDEN / f"kat_{stem}.json").read_text())


@pytest.fixture(scope="session")
def golden():
    return load_golden


@pytest.fixture(scope="session")
def kat():
    return load_kat
