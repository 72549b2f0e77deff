import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN_DIR = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box with -m gpu)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def load_golden(name):
    """Returns {key: torch tensor} for tests/golden/<name>.npz (16-bit floats restored from their bit patterns)."""
    z = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))
    out = {}
    for key in z.files:
        if key.endswith("_dtype"):
            continue
        if key.endswith("_bits16"):
            base = key[: -len("_bits16")]
            dt = {"torch.float16": torch.float16, "torch.bfloat16": torch.bfloat16}[str(z[base + "_dtype"])]
            out[base] = torch.from_numpy(np.array(z[key]).view(np.int16)).view(dt)
        else:
            out[key] = torch.from_numpy(np.array(z[key]))
    return out


@pytest.fixture(scope="session")
def golden():
    return load_golden
