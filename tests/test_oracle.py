"""Pins the CPU oracle (numpy and C) to the reference project's own vectors.

CPU only.  Sources of truth, by path inside the reference project:
  tests/inference/test_sage.py:46-63   closed-form fields of all 65536 code values
  tests/inference/test_sage.py:22-43   layout, byte count, unit-norm codebook, zero pad rows
  tests/golden/*                       outputs of the reference's synthetic_sage/decode_sage
"""

import hashlib

import numpy as np
import pytest
import torch

from oracle import c_oracle, sage_oracle
from sage_b200.synthetic import synthetic_sage

KEYS = ("packed_codes", "radius_codes", "radius_grid", "codebook", "permutation")


def sha(array) -> str:
    return hashlib.sha256(np.ascontiguousarray(array).tobytes()).hexdigest()


def to_numpy(packed):
    return {k: v.numpy() for k, v in packed.items()}


@pytest.mark.parametrize("seed,bits", [(0, 8), (1, 7), (2, 6)])
def test_discrete_fields_all_codes(seed, bits):
    """Every 16-bit code value with radius word 0xE4E4E4E4, against the closed form."""
    packed = to_numpy(synthetic_sage(128, 4096, seed=seed, permuted=False))
    assert packed["codebook"].shape[1] == 1 << bits
    words = np.arange(65536, dtype=np.int64).reshape(4096, 16)
    pairs = (words[:, ::2] | (words[:, 1::2] << 16)).astype(np.uint32).view(np.int32)
    packed["packed_codes"] = pairs.reshape(256, 1, 16, 8)
    packed["radius_codes"] = np.full_like(packed["radius_codes"], np.uint32(0xE4E4E4E4).view(np.int32))
    signs, index, radius = sage_oracle.unpack_fields(packed, 4096)
    expected_signs = 1 - 2 * ((words[..., None] >> np.arange(8)) & 1)
    np.testing.assert_array_equal(signs.reshape(4096, 16, 8), expected_signs)
    np.testing.assert_array_equal(index.reshape(4096, 16), (words >> 8) & ((1 << bits) - 1))
    np.testing.assert_array_equal(
        radius.reshape(4096, 16), (words >> (8 + bits)) | ((np.arange(16) % 4) << (8 - bits))
    )
    # the C oracle decodes the same table identically to the numpy oracle
    np.testing.assert_array_equal(
        c_oracle.decode_fp16(packed, 4096).view(np.uint16),
        sage_oracle.decode_fp16(packed, 4096).view(np.uint16),
    )


@pytest.mark.parametrize("k,n", [(128, 1), (256, 17), (2560, 9), (9728, 32), (16384, 1)])
@pytest.mark.parametrize("permuted", [False, True])
@pytest.mark.parametrize("seed,entries", [(0, 256), (1, 128), (2, 64)])
def test_layout_invariants(k, n, permuted, seed, entries):
    packed = synthetic_sage(k, n, seed=seed, permuted=permuted)
    again = synthetic_sage(k, n, seed=seed, permuted=permuted)
    assert packed["codebook"].shape == (4, entries, 2)
    assert packed["packed_codes"].shape == ((n + 15) // 16, k // 128, 16, 8)
    assert packed["radius_codes"].shape == ((n + 15) // 16, k // 128, 16)
    assert packed["radius_grid"].shape == ((n + 15) // 16, k // 128, 16, 2)
    assert packed["packed_codes"].dtype == packed["radius_codes"].dtype == torch.int32
    assert packed["radius_grid"].dtype == packed["codebook"].dtype == torch.float16
    total = sum(t.numel() * t.element_size() for t in packed.values())
    assert total == sage_oracle.packed_nbytes(n, k, entries, permuted)
    for key in KEYS:
        assert torch.equal(packed[key], again[key])
    if permuted:
        assert torch.equal(packed["permutation"].sort().values, torch.arange(k).int())
    book = packed["codebook"].permute(1, 0, 2).flatten(1).float()
    torch.testing.assert_close(book.norm(dim=-1), torch.ones(entries), rtol=5e-4, atol=0)
    assert torch.all(book >= 0)
    padded = (n + 15) // 16 * 16
    dense = sage_oracle.decode(to_numpy(packed), padded)
    assert np.count_nonzero(dense[n:]) == 0


def test_golden_small_cases(golden_cases):
    """Generator, numpy oracle and C oracle against the reference's own outputs."""
    assert len(golden_cases) >= 8
    for case in golden_cases:
        k, n = case["k"], case["n"]
        mine = synthetic_sage(k, n, seed=case["seed"], permuted=case["permuted"])
        for key in KEYS:
            got = mine[key].numpy()
            got = got.view(np.uint16) if got.dtype == np.float16 else got
            np.testing.assert_array_equal(got, case[key], err_msg=f"{case['name']}/{key}")
        packed = case["packed"]
        signs, index, radius = sage_oracle.unpack_fields(packed, n)
        np.testing.assert_array_equal(index, case["field_index"])
        np.testing.assert_array_equal(radius, case["field_radius"])
        sign_bits = ((signs < 0).astype(np.int64) << np.arange(8)).sum(-1)
        np.testing.assert_array_equal(sign_bits, case["field_sign_bits"])
        want = case["weight_fp16_bits"]
        np.testing.assert_array_equal(sage_oracle.decode_fp16(packed, n).view(np.uint16), want)
        np.testing.assert_array_equal(c_oracle.decode_fp16(packed, n).view(np.uint16), want)
        x = case["x_fp16_bits"].view(np.float16)
        y = case["y_fp32"]
        for got in (sage_oracle.linear_fp32(x, packed, n), c_oracle.linear_fp32(x, packed, n)):
            metrics = sage_oracle.error_metrics(got, y)
            # FP32 matmuls that differ only in summation order
            assert metrics["relative_l2"] < 2e-6, (case["name"], metrics)


def test_golden_hashes_benchmark_shapes(golden_hashes):
    """Benchmark-sized shapes: buffers and decoded weights by SHA-256."""
    for case in golden_hashes:
        k, n = case["k"], case["n"]
        packed = synthetic_sage(k, n, seed=case["seed"], permuted=case["permuted"])
        assert packed["codebook"].shape[1] == case["entries"]
        for key in KEYS:
            assert sha(packed[key].numpy().view(np.uint8)) == case["packed_sha256"][key], key
        weight = c_oracle.decode_fp16(packed, n)
        assert sha(weight.view(np.uint16)) == case["weight_fp16_sha256"]
        x = torch.randn(1, k, generator=torch.Generator().manual_seed(43), dtype=torch.float16)
        y = c_oracle.linear_fp32(x, packed, n)
        np.testing.assert_allclose(y[0, :8], case["y_fp32_first8"], rtol=2e-4, atol=2e-5)
        assert abs(float(np.linalg.norm(y)) - case["y_fp32_norm"]) < 1e-4 * case["y_fp32_norm"]


def test_numpy_and_c_oracle_agree_bitwise():
    for k, n, seed, permuted in [(384, 40, 0, True), (1280, 23, 1, False), (640, 64, 2, True)]:
        packed = to_numpy(synthetic_sage(k, n, seed=seed, permuted=permuted))
        a = sage_oracle.decode_fp16(packed, n).view(np.uint16)
        b = c_oracle.decode_fp16(packed, n).view(np.uint16)
        np.testing.assert_array_equal(a, b)
        q = c_oracle.decode_fp16(packed, n, apply_permutation=False).view(np.uint16)
        np.testing.assert_array_equal(
            q, sage_oracle.decode_fp16_quantised_order(packed, n).view(np.uint16)
        )


def test_zero_step_and_zero_grid_groups():
    """Constant grids give constant radii; a zero grid decodes to exact zeros
    (the reference checks this on its kernels at tests/inference/test_sage.py:158-171)."""
    packed = synthetic_sage(256, 17, seed=0)
    packed["radius_grid"][..., 1].zero_()
    packed["radius_grid"][..., 0].fill_(0.25)
    packed["radius_grid"][0, :, 0].zero_()
    assert np.count_nonzero(c_oracle.decode_fp16(packed, 17)[0]) == 0
    weight = c_oracle.decode_fp16(packed, 17, apply_permutation=False)
    norms = np.linalg.norm(weight[1:].astype(np.float32).reshape(16, -1, 8), axis=-1)
    np.testing.assert_allclose(norms, 0.25, rtol=2e-3)


def test_fp16_conversion_exhaustive():
    """The C oracle's half<->float helpers over all 65536 half values (identity grid)."""
    # a one-entry-style probe: decode with radius 1 reproduces the codebook values
    packed = to_numpy(synthetic_sage(128, 16, seed=2, permuted=False))
    packed["radius_grid"][..., 0] = np.float16(1.0)
    packed["radius_grid"][..., 1] = np.float16(0.0)
    a = sage_oracle.decode_fp16(packed, 16).view(np.uint16)
    b = c_oracle.decode_fp16(packed, 16).view(np.uint16)
    np.testing.assert_array_equal(a, b)
    # subnormal and rounding edges through tiny radii
    for scale in (2.0**-14, 2.0**-20, 3.0e-6, 6.0e-8, 1000.0):
        packed["radius_grid"][..., 0] = np.float16(scale)
        a = sage_oracle.decode_fp16(packed, 16).view(np.uint16)
        b = c_oracle.decode_fp16(packed, 16).view(np.uint16)
        np.testing.assert_array_equal(a, b)
