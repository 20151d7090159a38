"""Shared pytest set-up: the ``gpu`` marker, import path and small helpers."""

from __future__ import annotations

import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = Path(__file__).resolve().parent / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def golden():
    def load(name: str):
        return torch.load(GOLDEN / f"{name}.pt", map_location="cpu", weights_only=False)

    return load


@pytest.fixture()
def device():
    return torch.device("cuda", 0)


@pytest.fixture()
def status_clean():
    """Yield, then assert that no kernel of the test left a bit in the device status word."""

    from mini_inference_engine_b200 import _lib

    yield
    if torch.cuda.is_available():
        word = _lib.status_word(torch.device("cuda", 0))
        bits = int(word.item())
        word.zero_()
        assert bits == 0, f"device status word {bits}"
