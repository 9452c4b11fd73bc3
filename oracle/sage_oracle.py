"""CPU oracle for the SAGE packed-weight matmul.  TEST INFRASTRUCTURE ONLY.

This file restates, in numpy, the arithmetic the reference project defines for
its packed SAGE linear.  It exists so the CUDA kernels can be checked; it is
never imported by the `sage_b200` package, and the product path has no CPU
fallback.  Only the test-suite, the smoke check and the CPU-baseline leg of the
benchmark may import it.

Parity status: PINNED.  `tests/test_oracle.py` checks this file against
  * the reference's closed-form known-answer test over all 65536 code values
    (tests/inference/test_sage.py:46-63 in the reference project),
  * the reference's layout/byte-count/pad-row invariants
    (tests/inference/test_sage.py:22-43),
  * golden vectors produced by importing the reference's own Python decoder
    (`tests/golden/make_golden.py` is the generating script).

Reference sources followed, by path inside the reference project:
  tests/inference/reference.py:25-36   unpack_sage   -> `unpack_fields`
  tests/inference/reference.py:39-49   decode_sage   -> `decode`
  tests/inference/test_sage.py:113-115 FP16 dense QDQ contract -> `decode_fp16`
  tests/inference/test_sage.py:11-19   output gate   -> `error_metrics`
  csrc/sage/sage_gemm_cuda.cu:117-131  kernel-side dequantisation arithmetic
  weight_vq/sphquant/packing.py:43-75  bit layout written by the exporter

Packed layout (tiles = ceil(N/16), groups = K/128, E in {64,128,256}, D = log2 E):
  packed_codes int32 [tiles, groups, 16, 8]  two 16-bit codes per word
  radius_codes int32 [tiles, groups, 16]     sixteen 2-bit high radius fields
  radius_grid  fp16  [tiles, groups, 16, 2]  (min, step)
  codebook     fp16  [4, E, 2]               plane p holds dims (2p, 2p+1)
  permutation  int32 [K] or [0]              x_q[j] = x[perm[j]]
A 16-bit code is: bits 0-7 sign of dims 0-7 (1 = negative), bits 8..8+D-1 the
direction index, bits 8+D..15 the low 8-D radius bits.
"""

from __future__ import annotations

import numpy as np

PACKED_KEYS = ("packed_codes", "radius_codes", "radius_grid", "codebook", "permutation")


def as_numpy_packed(packed) -> dict[str, np.ndarray]:
    """Accept a dict of numpy arrays or torch CPU tensors; return numpy views."""
    out = {}
    for key in PACKED_KEYS:
        value = packed[key]
        if hasattr(value, "detach"):
            value = value.detach().cpu().numpy()
        out[key] = np.ascontiguousarray(value)
    return out


def unpack_fields(packed, n: int):
    """Split the packed words into (signs[+1/-1], direction index, radius code).

    Follows tests/inference/reference.py:25-36.  Returned arrays are indexed
    [row, group, vector(, dim)] in quantised channel order, rows cut to `n`.
    """
    p = as_numpy_packed(packed)
    codes = p["packed_codes"].astype(np.int64) & 0xFFFFFFFF
    tiles, groups = codes.shape[0], codes.shape[1]
    entries = p["codebook"].shape[1]
    dbits = entries.bit_length() - 1
    # [tiles, groups, 16, 8] -> [rows, groups, 8 words]
    words = codes.transpose(0, 2, 1, 3).reshape(tiles * 16, groups, 8)[:n]
    # word w holds vector 2w in its low half and vector 2w+1 in its high half
    vectors = np.stack((words & 0xFFFF, words >> 16), axis=-1).reshape(-1, groups, 16)
    bit = np.arange(8, dtype=np.int64)
    signs = 1 - 2 * ((vectors[..., None] >> bit) & 1)
    index = (vectors >> 8) & (entries - 1)
    low = vectors >> (8 + dbits)
    extra = p["radius_codes"].astype(np.int64) & 0xFFFFFFFF
    extra = extra.transpose(0, 2, 1).reshape(tiles * 16, groups)[:n]
    high = (extra[..., None] >> (2 * np.arange(16, dtype=np.int64))) & 3
    radius_code = low | (high << (8 - dbits))
    return signs, index, radius_code


def decode(packed, n: int) -> np.ndarray:
    """FP32 dequantised weight [n, K] in ORIGINAL channel order.

    Follows tests/inference/reference.py:39-49: radius = min + code * step in
    FP32, weight = sign * direction * radius in FP32, then the inverse of the
    input-channel gather (W[:, perm[j]] = W_q[:, j]).
    """
    p = as_numpy_packed(packed)
    signs, index, radius_code = unpack_fields(p, n)
    tiles, groups = p["packed_codes"].shape[0], p["packed_codes"].shape[1]
    entries = p["codebook"].shape[1]
    book = p["codebook"].transpose(1, 0, 2).reshape(entries, 8).astype(np.float32)
    grid = p["radius_grid"].transpose(0, 2, 1, 3).reshape(tiles * 16, groups, 2)[:n]
    grid = grid.astype(np.float32)
    radius = grid[..., 0, None] + radius_code.astype(np.float32) * grid[..., 1, None]
    radius = radius.astype(np.float32)
    weight = (signs.astype(np.float32) * book[index]) * radius[..., None]
    weight = weight.astype(np.float32).reshape(weight.shape[0], -1)
    perm = p["permutation"]
    if perm.size:
        original = np.empty_like(weight)
        original[:, perm.astype(np.int64)] = weight
        return original
    return weight


def decode_fp16(packed, n: int) -> np.ndarray:
    """The bit-exact dequantisation target: `decode(...)` rounded once to FP16.

    tests/inference/test_sage.py:113-115 in the reference: "the execution
    contract is native FP16 dense QDQ, not unrounded weights".
    """
    return decode(packed, n).astype(np.float16)


def decode_fp16_quantised_order(packed, n: int) -> np.ndarray:
    """FP16 weight with columns left in quantised (gathered) channel order."""
    p = dict(as_numpy_packed(packed))
    p["permutation"] = np.empty(0, dtype=np.int32)
    return decode(p, n).astype(np.float16)


def linear_fp32(x, packed, n: int) -> np.ndarray:
    """The reference CPU path: dequantise, round to FP16, matmul in FP32.

    tests/inference/test_sage.py:113-122 (`F.linear(x.float(), W.half().float())`).
    `x` is [..., K] FP16 (numpy or torch); the result is [..., n] float32.
    """
    if hasattr(x, "detach"):
        x = x.detach().cpu().numpy()
    w = decode_fp16(packed, n).astype(np.float32)
    x32 = np.asarray(x).astype(np.float32)
    return (x32.reshape(-1, x32.shape[-1]) @ w.T).reshape(*x32.shape[:-1], n)


def error_metrics(actual, expected) -> dict[str, float]:
    """relative L2 (= relative Frobenius) and max-abs, as the reference reports them
    (tests/inference/reference.py:208-213), plus max-abs over RMS
    (tests/inference/test_sage.py:11-19)."""
    a = np.asarray(actual, dtype=np.float64)
    e = np.asarray(expected, dtype=np.float64)
    err = a - e
    norm = max(float(np.linalg.norm(e)), 1e-30)
    rms = max(float(np.sqrt(np.mean(e * e))) if e.size else 0.0, 1e-30)
    max_abs = float(np.abs(err).max()) if err.size else 0.0
    return {
        "relative_l2": float(np.linalg.norm(err)) / norm,
        "max_absolute": max_abs,
        "max_absolute_over_rms": max_abs / rms,
    }


def packed_nbytes(n: int, k: int, entries: int, permuted: bool) -> int:
    """Byte-count identity from tests/inference/test_sage.py:32-34 (2.5 bit/weight)."""
    return (n + 15) // 16 * 16 * k * 5 // 16 + entries * 16 + (4 * k if permuted else 0)
