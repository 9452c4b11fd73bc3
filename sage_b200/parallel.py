"""Sharding SAGE-packed linears across GPUs (tensor parallelism).

The reference's packed inference is single-GPU; its only notion of column/row linears is
the tag table of the quantisation side (weight_vq/blockwise/artifacts.py:10-18: q/k/v/gate/up
are "col", o/down are "row").  This module applies those tags to the packed layout:

  column parallel  output rows are split in whole 16-row tiles: slice dim 0 of
                   packed_codes / radius_codes / radius_grid; codebook and permutation are
                   replicated; every rank sees the full input; no collective
  row parallel     input channels are split in whole 128-channel groups: slice dim 1 of the
                   three buffers; a rank's slice of the permutation must only reference the
                   rank's own channels (a block permutation, see `block_permutation`), so
                   that the rank can gather from its local activations; partial outputs are
                   summed with an all-reduce

Everything here is plain tensor slicing and runs on CPU tensors as well as CUDA tensors.
"""

from __future__ import annotations

import torch

PACKED_KEYS = ("packed_codes", "radius_codes", "radius_grid", "codebook", "permutation")


def block_permutation(in_features: int, blocks: int, seed: int, device="cpu") -> torch.Tensor:
    """A permutation of `in_features` channels that only permutes inside each of `blocks`
    equal contiguous blocks (each a multiple of 128 channels).  It is a legal SAGE
    `permutation` buffer, and any row-parallel split into a divisor of `blocks` ranks keeps
    every rank's gather inside its own slice of the activations."""
    if in_features % (128 * blocks):
        raise ValueError("each block must be a whole number of 128-channel groups")
    width = in_features // blocks
    gen = torch.Generator().manual_seed(seed)
    parts = [b * width + torch.randperm(width, generator=gen) for b in range(blocks)]
    return torch.cat(parts).to(torch.int32).to(device)


def shard_columns(packed: dict, out_features: int, rank: int, world: int) -> tuple[dict, int]:
    """Rank `rank`'s share of the output rows; returns (packed shard, local out_features)."""
    tiles = packed["packed_codes"].shape[0]
    if out_features % 16 or tiles % world:
        raise ValueError("column parallelism needs out_features to be a multiple of 16 * world")
    per = tiles // world
    lo, hi = rank * per, (rank + 1) * per
    shard = {
        "packed_codes": packed["packed_codes"][lo:hi].contiguous(),
        "radius_codes": packed["radius_codes"][lo:hi].contiguous(),
        "radius_grid": packed["radius_grid"][lo:hi].contiguous(),
        "codebook": packed["codebook"],
        "permutation": packed["permutation"],
    }
    return shard, per * 16


def shard_rows(packed: dict, rank: int, world: int) -> dict:
    """Rank `rank`'s share of the input channels (K / world of them, in quantised order).
    The permutation slice is re-based to index the rank's local activations."""
    groups = packed["packed_codes"].shape[1]
    if groups % world:
        raise ValueError("row parallelism needs K to be a multiple of 128 * world")
    per = groups // world
    lo, hi = rank * per, (rank + 1) * per
    permutation = packed["permutation"]
    if permutation.numel():
        local = permutation[lo * 128 : hi * 128].to(torch.int64) - lo * 128
        if int(local.min()) < 0 or int(local.max()) >= per * 128:
            raise ValueError(
                "the permutation mixes channels of different ranks; row parallelism needs a block "
                "permutation (see block_permutation) or an all-gather of the activations"
            )
        permutation = local.to(torch.int32).contiguous()
    return {
        "packed_codes": packed["packed_codes"][:, lo:hi].contiguous(),
        "radius_codes": packed["radius_codes"][:, lo:hi].contiguous(),
        "radius_grid": packed["radius_grid"][:, lo:hi].contiguous(),
        "codebook": packed["codebook"],
        "permutation": permutation,
    }


def row_parallel_input(x: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """The slice of the (original-order) activations a row-parallel rank consumes."""
    k = x.shape[-1]
    per = k // world
    return x[..., rank * per : (rank + 1) * per].contiguous()


def shard_vocab(table: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """Rows [rank*V/world, (rank+1)*V/world) of an FP16 [V, hidden] head matrix."""
    vocab = table.shape[0]
    if vocab % world:
        raise ValueError("the vocabulary must divide by the world size")
    per = vocab // world
    return table[rank * per : (rank + 1) * per].contiguous()
