"""Shared pytest set-up: the `gpu` marker, the repository on `sys.path`, and
loaders for the committed golden fixtures."""

from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

TESTS = Path(__file__).resolve().parent
if str(TESTS) not in sys.path:
    sys.path.insert(0, str(TESTS))  # helper modules beside the tests (checkpoint_cases, decoder_util)

GOLDEN = Path(__file__).resolve().parent / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def _nested(npz) -> dict:
    tree: dict = {}
    for key in npz.files:
        node = tree
        parts = key.split("/")
        for part in parts[:-1]:
            node = node.setdefault(part, {})
        node[parts[-1]] = npz[key]
    return tree


@pytest.fixture(scope="session")
def golden_quantizer() -> dict:
    return _nested(np.load(GOLDEN / "quantizer.npz"))


@pytest.fixture(scope="session")
def golden_linear() -> dict:
    return _nested(np.load(GOLDEN / "linear.npz"))
