"""Shared test configuration: the ``gpu`` marker and loaders for the golden vectors."""

import json
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
GOLDEN = Path(__file__).resolve().parent / "golden"
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config: pytest.Config) -> None:
    config.addinivalue_line("markers", "gpu: needs a CUDA device and the built CUDA library")


def pytest_collection_modifyitems(config: pytest.Config, items: list) -> None:
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="needs a CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def golden_meta() -> dict:
    return json.loads((GOLDEN / "golden.json").read_text())


@pytest.fixture(scope="session")
def golden_codecs() -> dict:
    with np.load(GOLDEN / "codecs.npz") as data:
        return {key: data[key] for key in data.files}


@pytest.fixture(scope="session")
def golden_transforms() -> dict:
    with np.load(GOLDEN / "transforms.npz") as data:
        return {key: data[key] for key in data.files}


@pytest.fixture(scope="session")
def golden_bitstream() -> dict:
    with np.load(GOLDEN / "bitstream.npz") as data:
        return {key: data[key] for key in data.files}
