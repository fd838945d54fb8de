"""Shared test plumbing: the ``gpu`` marker, import of the package (its folder
name has a hyphen, so it is loaded under the alias ``fastwamjoint_quantization_b200``)
and of the CPU oracle."""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import __graft_entry__ as entry  # noqa: E402

PKG = entry.load_package()


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def oracle():
    sys.path.insert(0, str(ROOT / "oracle"))
    import steerquant_oracle
    return steerquant_oracle


@pytest.fixture(scope="session")
def golden():
    data = np.load(ROOT / "tests" / "golden" / "steerquant_golden.npz")

    class Golden:
        def __getitem__(self, key):
            return torch.from_numpy(data[key])

        def bf16(self, key):
            return torch.from_numpy(data[key + "_bf16"]).view(torch.bfloat16)

    return Golden()


@pytest.fixture(scope="session")
def pkg():
    return PKG
