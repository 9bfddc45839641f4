"""Shared pytest configuration: the `gpu` marker, deterministic seeding, repo on sys.path."""

import hashlib
import pathlib
import sys

import pytest
import torch

ROOT = pathlib.Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(autouse=True)
def _seed(request):
    """Seed from the test id, as the reference's harness does (tests/conftest.py:81-93)."""
    digest = hashlib.sha256(request.node.nodeid.encode()).digest()
    torch.manual_seed(int.from_bytes(digest[:4], "little"))
    yield


@pytest.fixture(scope="session")
def golden():
    import numpy as np

    folder = ROOT / "tests" / "golden"
    return {p.stem: np.load(p, allow_pickle=False) for p in folder.glob("*.npz")}
