import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = ROOT / "tests" / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


class GoldenCases:
    """npz written by tests/golden/make_golden.py, grouped as {case: {field: array}}."""

    def __init__(self, path):
        flat = np.load(path)
        self.cases = {}
        for key in flat.files:
            case, _, field = key.partition("/")
            self.cases.setdefault(case, {})[field] = flat[key]

    def __iter__(self):
        return iter(self.cases.items())

    def __getitem__(self, name):
        return self.cases[name]


@pytest.fixture(scope="session")
def quant_golden():
    return GoldenCases(GOLDEN / "quant_cases.npz")


@pytest.fixture(scope="session")
def rmsnorm_golden():
    return GoldenCases(GOLDEN / "rmsnorm_cases.npz")


@pytest.fixture(scope="session")
def layer_golden():
    return dict(np.load(GOLDEN / "layer_cases.npz"))


@pytest.fixture(scope="session")
def built_library():
    """The CUDA library, (re)built in-tree if a source is newer than it."""
    from fp4_post_b200.build import build
    return build()
