"""Shared fixtures: marker registration, golden archives, import paths."""

from __future__ import annotations

import json
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]
GOLDEN = ROOT / "tests" / "golden"
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a); run with -m gpu on a B200")


class Archive:
    """A golden ``.npz`` viewed as ``case.field -> torch tensor``."""

    def __init__(self, path: Path):
        self._data = np.load(path)

    def __call__(self, key: str) -> torch.Tensor:
        return torch.from_numpy(np.asarray(self._data[key]))

    def has(self, key: str) -> bool:
        return key in self._data.files

    def int(self, key: str) -> int:
        return int(self._data[key])


@pytest.fixture(scope="session")
def golden():
    def load(name: str):
        path = GOLDEN / name
        if name.endswith(".json"):
            return json.loads(path.read_text())
        return Archive(path)

    return load


@pytest.fixture(scope="session")
def device():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")
