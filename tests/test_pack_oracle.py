"""CPU: the packing oracle against golden vectors made by the reference's own exporter
(tests/golden/make_golden_pack.py), and the packed result decoded by the SAGE oracle against
the exporter's contract (reference tests/inference/test_spherical_export.py:30-80)."""

import json
import pathlib

import numpy as np
import pytest

from oracle import pack_oracle, sage_oracle

GOLDEN = pathlib.Path(__file__).resolve().parent / "golden" / "pack_cases.npz"


def load_cases():
    data = np.load(GOLDEN)
    cases = []
    for meta in json.loads(bytes(data["index_json"]).decode()):
        case = dict(meta)
        prefix = meta["name"] + "/"
        for key in data.files:
            if key.startswith(prefix):
                case[key[len(prefix):]] = data[key]
        cases.append(case)
    return cases


CASES = load_cases()


def packed_of(case):
    packed = {key.split("/", 1)[1]: value for key, value in case.items() if key.startswith("packed/")}
    for key in ("radius_grid", "codebook", "radius_scales", "radius_mins"):
        if key in packed:
            packed[key] = packed[key].view(np.float16)
    return packed


@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
def test_oracle_reproduces_the_reference_exporter(case):
    want = packed_of(case)
    got = pack_oracle.pack_radii(case["state/signs"], case["state/direction_indices"], case["radius"],
                                 1 << case["bits"], case["sage"])
    for key, value in got.items():
        assert value.dtype == want[key].dtype and value.shape == want[key].shape, key
        np.testing.assert_array_equal(value.view(np.uint8), want[key].view(np.uint8), err_msg=key)


@pytest.mark.parametrize("case", [c for c in CASES if c["sage"]], ids=[c["name"] for c in CASES if c["sage"]])
def test_packed_sage_decodes_to_signs_directions_radii(case):
    """pack -> decode is exact: signs * codebook[index] * (min + code * step), channels back in
    original order, pad rows zero (rtol = 0, atol = 0 as in the reference's test)."""
    packed, n, k = packed_of(case), case["n"], case["k"]
    signs, indices, codes = sage_oracle.unpack_fields(packed, n)
    assert np.array_equal(signs.reshape(n, k), case["state/signs"])
    assert np.array_equal(indices.reshape(n, -1), case["state/direction_indices"])
    grid = packed["radius_grid"].transpose(0, 2, 1, 3).reshape(-1, k // 128, 2)[:n].astype(np.float32)
    radii = grid[..., 0:1] + codes.reshape(n, -1, 16).astype(np.float32) * grid[..., 1:2]
    assert np.count_nonzero(grid[0, :, 1]) == 0  # constant and underflowing groups: zero step
    book = packed["codebook"].transpose(1, 0, 2).reshape(-1, 8).astype(np.float32)
    expected = (case["state/signs"].reshape(n, -1, 8) * book[case["state/direction_indices"]]
                * radii.reshape(n, -1)[..., None]).reshape(n, k)
    expected = expected[:, case["state/channel_unpermutation"]]
    np.testing.assert_array_equal(sage_oracle.decode(packed, n), expected.astype(np.float32))
    assert np.count_nonzero(packed["packed_codes"][-1, :, n % 16:]) == 0 or n % 16 == 0
    assert bool(packed["permutation"].size) == case["permuted"]
