"""Shared fixtures: the gpu marker, golden vectors and the reference's shipped codebooks."""

import json
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
GOLDEN = ROOT / "tests" / "golden"
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def _load_tables():
    raw = json.loads((GOLDEN / "shipped_codebooks.json").read_text())
    out = {}
    for key, v in raw.items():
        d, b = key[1:].split("_b")
        c = np.array([int(h, 16) for h in v["centroids"]], dtype=np.uint32).view(np.float32)
        bd = np.array([int(h, 16) for h in v["boundaries"]], dtype=np.uint32).view(np.float32)
        out[(int(d), int(b))] = (c, bd)
    return out


@pytest.fixture(scope="session")
def tables():
    """(d, bits) -> (centroids, boundaries), float32, exactly as the reference ships them."""
    return _load_tables()


@pytest.fixture(scope="session")
def golden():
    return np.load(GOLDEN / "reference_vectors.npz")


@pytest.fixture(scope="session")
def scenarios():
    return json.loads((GOLDEN / "cache_scenarios.json").read_text())


@pytest.fixture(scope="session")
def oracle():
    from oracle import tq_oracle
    return tq_oracle
