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

A checkpoint exported by the reference stores one GLOBAL permutation per matrix
(weight_vq/sphquant/packing.py:68-70), which mixes the channels of all ranks.  Two load-time
remedies keep such matrices row-parallel:

  fold (down_proj)   the permutation of down_proj's input moves into the ROW ORDER of gate_proj
                     and up_proj (`permute_output_rows`): SwiGLU is elementwise, so the MLP
                     then produces its intermediate activations directly in down_proj's
                     quantised channel order, down_proj needs no gather, and a contiguous
                     K split lines up with the column split of gate/up.  No extra exchange.
  gather (o_proj)    the attention output of all ranks is all-gathered (a few KB per token) and
                     each rank picks its K slice's source channels out of the full row
                     (`shard_rows_global` returns the index list); the shard itself carries no
                     permutation.

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


def permute_output_rows(packed: dict, out_features: int, order: torch.Tensor) -> dict:
    """The same packed linear with its output rows re-ordered: new row i = old row order[i]
    (`order` a permutation of range(out_features), out_features a multiple of 16).  Pure
    re-tiling of the three row-indexed buffers; codebook and permutation are shared."""
    tiles, groups = packed["packed_codes"].shape[:2]
    if out_features != tiles * 16 or order.numel() != out_features:
        raise ValueError("row re-ordering needs out_features = 16 * tiles and a full permutation")
    order = order.to(torch.int64).to(packed["packed_codes"].device)

    def rows_first(t):  # [tiles, groups, 16, ...] -> [tiles * 16, groups, ...]
        return t.transpose(1, 2).reshape(tiles * 16, groups, *t.shape[3:])

    def tiled(t):       # back to [tiles, groups, 16, ...]
        return t.reshape(tiles, 16, groups, *t.shape[2:]).transpose(1, 2).contiguous()

    return {
        "packed_codes": tiled(rows_first(packed["packed_codes"])[order]),
        "radius_codes": tiled(rows_first(packed["radius_codes"])[order]),
        "radius_grid": tiled(rows_first(packed["radius_grid"])[order]),
        "codebook": packed["codebook"],
        "permutation": packed["permutation"],
    }


def fold_input_permutation(producers: list[tuple[dict, int]], consumer: dict) -> tuple[list[dict], dict]:
    """Move `consumer`'s input permutation into the output-row order of the packed linears that
    (through an elementwise function) produce its input: returns (re-ordered producers, the
    consumer with an empty permutation).  y = consumer(f(producers(x))) is unchanged."""
    permutation = consumer["permutation"]
    if permutation.numel() == 0:
        return [p for p, _ in producers], consumer
    folded = [permute_output_rows(p, n, permutation) for p, n in producers]
    plain = dict(consumer)
    plain["permutation"] = permutation[:0]
    return folded, plain


def shard_rows_global(packed: dict, rank: int, world: int) -> tuple[dict, torch.Tensor]:
    """Row-parallel share under ANY permutation: the rank's K / world quantised channels, plus
    the source channel (in the full activation row) of each of them.  The shard carries no
    permutation; the caller gathers x_full[..., index] itself (after an all-gather when the
    activations are spread over the ranks)."""
    groups = packed["packed_codes"].shape[1]
    if groups % world:
        raise ValueError("row parallelism needs K to be a multiple of 128 * world")
    per = groups // world
    lo, hi = rank * per, (rank + 1) * per
    permutation = packed["permutation"]
    k = groups * 128
    if permutation.numel():
        index = permutation[lo * 128 : hi * 128].to(torch.int64)
    else:
        index = torch.arange(lo * 128, hi * 128, device=permutation.device)
    shard = {
        "packed_codes": packed["packed_codes"][:, lo:hi].contiguous(),
        "radius_codes": packed["radius_codes"][:, lo:hi].contiguous(),
        "radius_grid": packed["radius_grid"][:, lo:hi].contiguous(),
        "codebook": packed["codebook"],
        "permutation": permutation[:0],
    }
    assert int(index.max()) < k
    return shard, index


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
