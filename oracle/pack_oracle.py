"""CPU oracle for the export-side packing of spherical linears.  TEST INFRASTRUCTURE ONLY.

Restates, in numpy, the tensor program of the reference's exporter from the radii on
(weight_vq/sphquant/packing.py:32-75 in the reference project): grid fitting against an FP16
(min, step), radius-code selection, sign / index / radius bit packing, SAGE's tiling and row
padding, SPHQuant's row-major form.  Never imported by the `sage_b200` package.

Parity status: PINNED.  `tests/test_pack_oracle.py` checks this file against golden vectors
produced by running the reference's own `pack_spherical` (`tests/golden/make_golden_pack.py`
is the generating script; the one function the exporter imports from an un-vendored training
package, `direction_codebook_from_logits`, is supplied there from the reference's own patch,
patches/paroquant/0002-...patch:368-389).
"""

from __future__ import annotations

import numpy as np


def pack_radii(signs: np.ndarray, indices: np.ndarray, radius: np.ndarray, entries: int, sage: bool) -> dict:
    """signs int8 [n, k] (+1/-1), indices [n, k/8], FP32 radii [n, k/8] -> packed buffers."""
    n, k = signs.shape
    groups = k // 128
    bits = entries.bit_length() - 1
    levels = (1 << (10 - bits)) - 1
    low_bits = 8 - bits
    radius = radius.astype(np.float32).reshape(n, groups, 16)
    minimum32 = radius.min(axis=-1)                                              # packing.py:35
    step = ((radius.max(axis=-1) - minimum32) / np.float32(levels)).astype(np.float16)  # :36
    minimum = minimum32.astype(np.float16)                                       # :37
    live = step > 0
    safe = np.where(live, step.astype(np.float32), np.float32(1))                # :38
    codes = np.rint((radius - minimum.astype(np.float32)[..., None]) / safe[..., None])  # :39
    codes = np.clip(codes, 0, levels).astype(np.int64)                           # :40
    codes = np.where(live[..., None], codes, 0)                                  # :41
    negative = (signs.reshape(n, groups, 16, 8) < 0).astype(np.int64)            # :43
    sign_words = (negative << np.arange(8)).sum(-1)                              # :44
    words = (sign_words | (indices.astype(np.int64).reshape(n, groups, 16) << 8)
             | ((codes & ((1 << low_bits) - 1)) << (8 + bits)))                  # :46-50
    high = ((codes >> low_bits) << (2 * np.arange(16))).sum(-1)                  # :51
    if not sage:                                                                 # :52-59
        return {
            "packed_codes": words.reshape(n, k // 8).astype(np.uint16).view(np.int16),
            "radius_extra": high.astype(np.uint32).view(np.int32),
            "radius_scales": step,
            "radius_mins": minimum,
        }
    pairs = words[..., 0::2] | (words[..., 1::2] << 16)                          # :62
    grid = np.stack((minimum, step), axis=-1)                                    # :63
    padding = (-n) % 16                                                          # :64-67
    pairs = np.pad(pairs, ((0, padding), (0, 0), (0, 0)))
    high = np.pad(high, ((0, padding), (0, 0)))
    grid = np.pad(grid, ((0, padding), (0, 0), (0, 0)))
    return {                                                                     # :71-75
        "packed_codes": np.ascontiguousarray(
            pairs.reshape(-1, 16, groups, 8).transpose(0, 2, 1, 3)).astype(np.uint32).view(np.int32),
        "radius_codes": np.ascontiguousarray(
            high.reshape(-1, 16, groups).transpose(0, 2, 1)).astype(np.uint32).view(np.int32),
        "radius_grid": np.ascontiguousarray(grid.reshape(-1, 16, groups, 2).transpose(0, 2, 1, 3)),
    }
