"""The SPHQuant oracle against golden vectors made by the reference's own Python
(tests/golden/make_golden_sph.py), and this repo's generator against the same files."""

import hashlib
import json
import pathlib

import numpy as np
import pytest

from oracle import sph_oracle
from sage_b200.synthetic import synthetic_sphquant

GOLDEN = pathlib.Path(__file__).parent / "golden"
KEYS = sph_oracle.KEYS


def load_cases():
    data = np.load(GOLDEN / "sph_cases.npz")
    index = json.loads(bytes(data["index_json"]).decode())
    return data, index


def packed_of(data, name):
    packed = {key: data[f"{name}/{key}"] for key in KEYS}
    for key in ("radius_scales", "radius_mins", "codebook"):
        packed[key] = packed[key].view(np.float16)
    return packed


def test_decode_matches_reference_bits():
    data, index = load_cases()
    for case in index:
        packed = packed_of(data, case["name"])
        weight = sph_oracle.decode(packed)
        assert weight.shape == (case["n"], case["k"])
        assert np.array_equal(weight.view(np.uint32), data[f"{case['name']}/weight_fp32"].view(np.uint32)), case


def test_linear_matches_reference_output():
    data, index = load_cases()
    for case in index:
        name = case["name"]
        x = data[f"{name}/x_fp16_bits"].view(np.float16)
        y = sph_oracle.linear_fp32(x, packed_of(data, name))
        want = data[f"{name}/y_fp32"]
        assert np.linalg.norm(y - want) <= 1e-6 * np.linalg.norm(want) + 1e-12


def test_field_layout_closed_form():
    """Every 16-bit code under radius word 0xE4E4E4E4 (fields 0,1,2,3 repeating), the check the
    reference applies to its SAGE fields (tests/inference/test_sage.py:46-63), here for the
    SPHQuant bit split: signs bits 0-7, index bits 8-13, radius = bits 14-15 | high << 2."""
    codes = np.arange(65536, dtype=np.uint16).view(np.int16).reshape(32, 2048)
    packed = {
        "packed_codes": codes,
        "radius_extra": np.full((32, 128), 0xE4E4E4E4, dtype=np.uint32).view(np.int32),
        "radius_scales": np.ones((32, 128), np.float16), "radius_mins": np.zeros((32, 128), np.float16),
        "codebook": np.ones((64, 8), np.float16),
    }
    signs, index, radius = sph_oracle.unpack_fields(packed)
    words = np.arange(65536).reshape(32, 2048)
    vector = np.arange(2048) % 16
    assert np.array_equal(index, (words >> 8) & 63)
    assert np.array_equal(radius, (words >> 14) | ((vector % 4) << 2)[None, :])
    assert np.array_equal(signs, 1 - 2 * ((words[..., None] >> np.arange(8)) & 1))


@pytest.mark.parametrize("case", json.loads((GOLDEN / "sph_hashes.json").read_text())["cases"],
                         ids=lambda c: f"k{c['k']}_n{c['n']}_s{c['seed']}")
def test_generator_and_decode_hashes(case):
    def sha(array):
        return hashlib.sha256(np.ascontiguousarray(array).tobytes()).hexdigest()

    packed = synthetic_sphquant(case["k"], case["n"], case["seed"])
    for key in KEYS:
        assert sha(packed[key].numpy().view(np.uint8)) == case["packed_sha256"][key], key
    weight = sph_oracle.decode(packed)
    assert sha(weight.view(np.uint32)) == case["weight_fp32_sha256"]
    assert sha(weight.astype(np.float16).view(np.uint16)) == case["weight_fp16_sha256"]
