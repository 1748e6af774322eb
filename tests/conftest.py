"""pytest configuration: the ``gpu`` marker, repo root on sys.path, shared helpers."""
from __future__ import annotations

import json
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN_DIR = Path(__file__).resolve().parent / "golden"


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
def golden_small():
    return torch.load(GOLDEN_DIR / "golden_small.pt")


@pytest.fixture(scope="session")
def golden_hashes():
    return json.loads((GOLDEN_DIR / "golden_hashes.json").read_text())


@pytest.fixture(scope="session")
def same_cpu_as_golden(golden_hashes):
    """True when this host evaluates torch CPU ops exactly like the host that made the
    fixtures (same torch build and vector ISA); bit-for-bit checks are only demanded then,
    other hosts check to one unit in the last place."""
    meta = golden_hashes["meta"]
    return (meta["torch"] == torch.__version__
            and meta["cpu_capability"] == torch.backends.cpu.get_cpu_capability())
