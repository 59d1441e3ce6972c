"""Shared test set-up: marker registration, import paths, fixture loading, GPU gating."""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = Path(__file__).resolve().parent / "golden" / "reference_vectors.npz"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def golden():
    """Vectors produced by the reference package (tests/golden/make_fixtures.py)."""
    with np.load(GOLDEN, allow_pickle=False) as data:
        return {name: data[name] for name in data.files}


@pytest.fixture(scope="session")
def pkg():
    import strix_halo_int4_gemms_b200 as package

    return package


@pytest.fixture(scope="session")
def native_lib(pkg):
    """The built CUDA library; building is part of the test session when it is stale."""
    import importlib.util

    spec = importlib.util.spec_from_file_location("b200_build", ROOT / "strix-halo-int4-gemms_b200" / "build.py")
    build = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(build)
    return build.build_native()
