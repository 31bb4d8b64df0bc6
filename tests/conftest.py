import json
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = ROOT / "tests" / "golden" / "canon_golden.npz"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


class GoldenCase:
    """One case of tests/golden/canon_golden.npz with tensors restored to their dtype."""

    def __init__(self, meta, z):
        self.meta = meta
        self.name = meta["name"]
        self.dtype = getattr(torch, meta["dtype"])
        self._z = z

    def has(self, key):
        return f"{self.name}.{key}" in self._z.files

    def get(self, key):
        arr = self._z[f"{self.name}.{key}"]
        if arr.dtype == np.uint16:
            return torch.from_numpy(arr.view(np.int16).copy()).view(torch.bfloat16)
        return torch.from_numpy(arr.copy())

    def __getattr__(self, key):
        if key in self.meta:
            return self.meta[key]
        raise AttributeError(key)

    def __repr__(self):
        m = self.meta
        return (f"{m['name']}[{m['dtype']} B{m['B']} T{m['T']} D{m['D']} K{m['K']} bias={m['bias']} "
                f"act={m['activation']} mask={m['mask']}]")


def load_golden(path=GOLDEN):
    z = np.load(path)
    meta = json.loads(bytes(z["meta"]).decode())
    return [GoldenCase(m, z) for m in meta]


GOLDEN_CASES = load_golden()
# gradients of the reference's CanonLayer (generator: tests/golden/make_bwd_golden.py)
GOLDEN_BWD_CASES = load_golden(ROOT / "tests" / "golden" / "canon_bwd_golden.npz")


@pytest.fixture(scope="session")
def golden_cases():
    return GOLDEN_CASES
