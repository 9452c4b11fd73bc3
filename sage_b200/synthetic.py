"""Seeded synthetic SAGE-packed weights (inputs for tests and benchmarks).

Produces the five packed buffers of one SAGE linear with the value
distributions of the reference's `synthetic_sage`
(weight_vq/checkpoint.py:54-89 in the reference project): the Adaptive Bit
Split is drawn from the seed (6, 7 or 8 direction bits, i.e. 64/128/256
codebook entries and 4/3/2 radius bits), the codebook is a row-normalised
U[0,1) matrix, every code/radius bit pattern is legal and drawn uniformly,
the (min, step) grid is U[0,1)*sqrt(8/K) with the step divided by the number
of radius levels minus one, pad rows of the last 16-row tile are zero, and the
input-channel permutation is a random permutation of K.

The draw order matches the reference generator, so for the same torch version
and seed the buffers are identical to the reference's; `tests/golden` pins that.
"""

from __future__ import annotations

import math

import torch

PACKED_KEYS = ("packed_codes", "radius_codes", "radius_grid", "codebook", "permutation")


def synthetic_sage(
    in_features: int,
    out_features: int,
    seed: int = 0,
    *,
    permuted: bool = True,
    direction_bits: int | None = None,
) -> dict[str, torch.Tensor]:
    """Return CPU tensors {packed_codes, radius_codes, radius_grid, codebook, permutation}.

    `direction_bits` (6, 7 or 8) forces the bit split; by default the seed
    chooses it exactly as the reference does (seed 0 -> 8, 1 -> 7, 2 -> 6).
    """
    if in_features <= 0 or in_features % 128 or out_features <= 0:
        raise ValueError("SAGE requires positive N and K divisible by 128")
    if direction_bits not in (None, 6, 7, 8):
        raise ValueError("direction_bits must be 6, 7 or 8")
    gen = torch.Generator().manual_seed(seed)
    drawn = int(torch.randint(6, 9, (), generator=gen))
    dbits = drawn if direction_bits is None else direction_bits
    entries = 1 << dbits
    levels = 1 << (10 - dbits)
    tiles = (out_features + 15) // 16
    groups = in_features // 128

    directions = torch.rand(entries, 8, generator=gen)
    directions = torch.nn.functional.normalize(directions, dim=-1)
    lo, hi = -(2**31), 2**31
    packed_codes = torch.randint(lo, hi, (tiles, groups, 16, 8), generator=gen, dtype=torch.int32)
    radius_codes = torch.randint(lo, hi, (tiles, groups, 16), generator=gen, dtype=torch.int32)
    radius_grid = torch.rand(tiles, groups, 16, 2, generator=gen) * math.sqrt(8 / in_features)
    radius_grid[..., 1] /= levels - 1
    tail = out_features % 16
    if tail:
        for buffer in (packed_codes, radius_codes, radius_grid):
            buffer[-1, :, tail:] = 0
    if permuted:
        permutation = torch.randperm(in_features, generator=gen, dtype=torch.int32)
    else:
        permutation = torch.empty(0, dtype=torch.int32)
    # plane p of the stored codebook holds dims (2p, 2p+1) of every entry
    codebook = directions.half().reshape(entries, 4, 2).permute(1, 0, 2).contiguous()
    return {
        "packed_codes": packed_codes,
        "radius_codes": radius_codes,
        "radius_grid": radius_grid.half(),
        "codebook": codebook,
        "permutation": permutation,
    }


def packed_to(packed: dict[str, torch.Tensor], device) -> dict[str, torch.Tensor]:
    return {key: value.to(device) for key, value in packed.items()}


def synthetic_sage_device(
    in_features: int,
    out_features: int,
    seed: int,
    device,
    *,
    permuted: bool = True,
    direction_bits: int | None = None,
) -> dict[str, torch.Tensor]:
    """Same distributions as `synthetic_sage`, drawn with the device's generator.

    For benchmarks that need hundreds of matrices quickly; the values differ from the
    CPU generator's (another random stream), the shapes, dtypes and distributions do not.
    """
    if in_features <= 0 or in_features % 128 or out_features <= 0:
        raise ValueError("SAGE requires positive N and K divisible by 128")
    dbits = direction_bits if direction_bits is not None else 6 + seed % 3
    entries = 1 << dbits
    levels = 1 << (10 - dbits)
    tiles = (out_features + 15) // 16
    groups = in_features // 128
    gen = torch.Generator(device=device).manual_seed(seed)
    lo, hi = -(2**31), 2**31
    directions = torch.nn.functional.normalize(
        torch.rand(entries, 8, generator=gen, device=device), dim=-1
    )
    packed_codes = torch.randint(lo, hi, (tiles, groups, 16, 8), generator=gen, device=device, dtype=torch.int32)
    radius_codes = torch.randint(lo, hi, (tiles, groups, 16), generator=gen, device=device, dtype=torch.int32)
    radius_grid = torch.rand(tiles, groups, 16, 2, generator=gen, device=device) * math.sqrt(8 / in_features)
    radius_grid[..., 1] /= levels - 1
    tail = out_features % 16
    if tail:
        for buffer in (packed_codes, radius_codes, radius_grid):
            buffer[-1, :, tail:] = 0
    if permuted:
        permutation = torch.randperm(in_features, generator=gen, device=device).int()
    else:
        permutation = torch.empty(0, dtype=torch.int32, device=device)
    return {
        "packed_codes": packed_codes,
        "radius_codes": radius_codes,
        "radius_grid": radius_grid.half(),
        "codebook": directions.half().reshape(entries, 4, 2).permute(1, 0, 2).contiguous(),
        "permutation": permutation,
    }


def linear_algorithmic_bytes(rows: int, n: int, k: int, entries: int, permuted: bool) -> int:
    """Bytes one packed-linear call must move: packed weight once (2.5 bit/weight over the
    padded rows), codebook, permutation, activations in and out."""
    padded = (n + 15) // 16 * 16
    return padded * k * 5 // 16 + 16 * entries + (4 * k if permuted else 0) + 2 * rows * k + 2 * rows * n


def synthetic_sphquant(in_features: int, out_features: int, seed: int = 0) -> dict[str, torch.Tensor]:
    """Seeded SPHQuant 64/4 buffers on the CPU, drawn in the order of the reference generator
    (weight_vq/checkpoint.py:35-51) so that equal seeds give equal bits: a unit-norm non-negative
    [64, 8] codebook, every 16-bit code pattern, every 32-bit high-radius word, FP16
    (scale, minimum) per (row, 128-channel group) sized for unit-variance outputs."""
    if in_features <= 0 or in_features % 128 or out_features <= 0:
        raise ValueError("SPHQuant requires positive N and K divisible by 128")
    gen = torch.Generator().manual_seed(seed)
    codebook = torch.nn.functional.normalize(torch.rand(64, 8, generator=gen), dim=-1).half()
    cells = (out_features, in_features // 128)
    unit = (8 / in_features) ** 0.5
    codes = torch.randint(-32768, 32768, (out_features, in_features // 8), generator=gen, dtype=torch.int16)
    extra = torch.randint(-(2**31), 2**31, cells, generator=gen, dtype=torch.int32)
    scales = (torch.rand(cells, generator=gen) * unit / 15).half()
    mins = (torch.rand(cells, generator=gen) * unit).half()
    return {"packed_codes": codes, "radius_extra": extra, "radius_scales": scales, "radius_mins": mins,
            "codebook": codebook}


def sph_algorithmic_bytes(rows: int, n: int, k: int) -> int:
    """HBM bytes one SPHQuant linear call has to move: packed buffers once, x and y."""
    return n * k // 4 + n * (k // 128) * 8 + 64 * 16 + 2 * rows * k + 2 * rows * n
