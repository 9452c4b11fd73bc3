"""Shared fixtures.  `gpu` marks tests that need a CUDA device and the built library."""

import json
import pathlib
import sys

import numpy as np
import pytest

ROOT = pathlib.Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = ROOT / "tests" / "golden"


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
def golden_cases():
    """Small reference-generated cases: list of dicts with packed buffers and outputs."""
    data = np.load(GOLDEN / "sage_cases.npz")
    index = json.loads(bytes(data["index_json"]).decode())
    cases = []
    for meta in index:
        name = meta["name"]
        case = dict(meta)
        for key in data.files:
            if key.startswith(name + "/"):
                case[key.split("/", 1)[1]] = data[key]
        case["packed"] = {
            "packed_codes": case["packed_codes"],
            "radius_codes": case["radius_codes"],
            "radius_grid": case["radius_grid"].view(np.float16),
            "codebook": case["codebook"].view(np.float16),
            "permutation": case["permutation"],
        }
        cases.append(case)
    return cases


@pytest.fixture(scope="session")
def golden_hashes():
    return json.loads((GOLDEN / "sage_hashes.json").read_text())["cases"]
