"""Shared test plumbing: the ``gpu`` marker, import paths and fixture loaders."""
from __future__ import annotations

import importlib.util
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
GOLDEN = ROOT / "tests" / "golden"
for p in (str(ROOT), str(ROOT / "oracle")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on the GPU box)")


def _load_make_golden():
    spec = importlib.util.spec_from_file_location("make_golden", GOLDEN / "make_golden.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


@pytest.fixture(scope="session")
def golden_inputs():
    """The seeded dense-input generators the fixtures were made from."""
    return _load_make_golden()


@pytest.fixture(scope="session")
def golden():
    def load(name: str):
        return dict(np.load(GOLDEN / f"{name}.npz"))
    return load


@pytest.fixture(scope="session")
def oracle():
    import gkv_oracle
    gkv_oracle.build()
    return gkv_oracle
