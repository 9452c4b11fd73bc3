"""CPU oracle for the SPHQuant 64/4 packed format (TEST INFRASTRUCTURE ONLY).

Only tests/, the smoke check and the bench's CPU baseline may import this module; the
product path never does.

Restates, in numpy, the reference's arithmetic decode of the format
(tests/inference/reference.py:8-22 in the reference project: `unpack_sphquant`,
`decode_sphquant`) and the kernel-side field layout
(csrc/sphquant/sph_gemv_cuda.cu:317-332):

  packed_codes  int16 [N][K/8]   one 16-bit code per 8-channel vector:
                                 bits 0-7 sign of dims 0-7 (1 = negative), bits 8-13 direction
                                 index (64 entries), bits 14-15 low two radius bits
  radius_extra  int32 [N][K/128] sixteen 2-bit fields, field v = high two radius bits of
                                 vector v of the group; radius code = low | high << 2 (0..15)
  radius_scales fp16  [N][K/128] radius = min + code * scale  (FP32)
  radius_mins   fp16  [N][K/128]
  codebook      fp16  [64][8]    unit-norm non-negative directions, entry-major

  W[n][8v + d] = sign * codebook[index][d] * radius      (FP32; `.astype(float16)` for the
                                                          dense FP16 weight)

Parity pinned: tests/test_sph_oracle.py checks this file against golden vectors produced by the
reference's own `synthetic_sphquant` and `decode_sphquant` (tests/golden/make_golden_sph.py).
"""

from __future__ import annotations

import numpy as np

KEYS = ("packed_codes", "radius_extra", "radius_scales", "radius_mins", "codebook")


def as_numpy(packed) -> dict[str, np.ndarray]:
    out = {}
    for key in KEYS:
        value = packed[key]
        out[key] = value.detach().cpu().numpy() if hasattr(value, "detach") else np.asarray(value)
    return out


def unpack_fields(packed):
    """(signs [N][K/8][8] in {+1,-1}, direction index [N][K/8], radius code [N][K/8])."""
    p = as_numpy(packed)
    words = p["packed_codes"].astype(np.int64) & 0xFFFF
    extra = p["radius_extra"].astype(np.int64) & 0xFFFFFFFF
    signs = 1 - 2 * ((words[..., None] >> np.arange(8)) & 1)
    index = (words >> 8) & 63
    high = (extra[..., None] >> (2 * np.arange(16))) & 3          # [N][groups][16]
    radius = (words >> 14) | (high.reshape(high.shape[0], -1) << 2)
    return signs, index, radius


def decode(packed) -> np.ndarray:
    """Dense FP32 weight [N][K] (reference decode_sphquant)."""
    p = as_numpy(packed)
    signs, index, radius = unpack_fields(p)
    directions = p["codebook"].astype(np.float32)[index]          # [N][K/8][8]
    mins = np.repeat(p["radius_mins"].astype(np.float32), 16, axis=1)
    scales = np.repeat(p["radius_scales"].astype(np.float32), 16, axis=1)
    radii = (mins + radius.astype(np.float32) * scales).astype(np.float32)
    weight = signs.astype(np.float32) * directions * radii[..., None]
    return weight.reshape(weight.shape[0], -1).astype(np.float32)


def decode_fp16(packed) -> np.ndarray:
    return decode(packed).astype(np.float16)


def linear_fp32(x, packed) -> np.ndarray:
    """y = x . W^T with the FP32 decoded weight (the reference tests' `expected`,
    tests/inference/test_ops.py:22)."""
    x32 = (x.detach().cpu().numpy() if hasattr(x, "detach") else np.asarray(x)).astype(np.float32)
    w = decode(packed)
    return (x32.reshape(-1, x32.shape[-1]) @ w.T).reshape(*x32.shape[:-1], w.shape[0])


def packed_nbytes(n: int, k: int) -> int:
    """Bytes of the five buffers: 2 bit/weight codes + 8 bytes per (row, group) + codebook."""
    return n * k // 4 + n * (k // 128) * 8 + 64 * 8 * 2
