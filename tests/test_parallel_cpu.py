"""Tensor-parallel sharding of packed linears, on CPU: shards recombine to the full matrix
under the oracle, and a world-size-2 gloo run reproduces the unsharded output with an
all-reduce (row parallel) and an all-gather (column parallel)."""

import os
import tempfile

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import c_oracle
from sage_b200.parallel import (block_permutation, fold_input_permutation, permute_output_rows, row_parallel_input,
                                shard_columns, shard_rows, shard_rows_global, shard_vocab)
from sage_b200.synthetic import synthetic_sage


def test_block_permutation_is_a_blockwise_permutation():
    perm = block_permutation(2048, 8, seed=3)
    assert perm.dtype == torch.int32 and perm.numel() == 2048
    assert torch.equal(perm.sort().values, torch.arange(2048, dtype=torch.int32))
    for b in range(8):
        block = perm[b * 256 : (b + 1) * 256]
        assert int(block.min()) == b * 256 and int(block.max()) == b * 256 + 255
    with pytest.raises(ValueError):
        block_permutation(1000, 8, seed=0)


@pytest.mark.parametrize("world", [2, 4])
def test_column_shards_recombine(world):
    k, n = 512, 128
    packed = synthetic_sage(k, n, seed=1)
    full = c_oracle.decode_fp16(packed, n)
    parts = []
    for rank in range(world):
        shard, local_n = shard_columns(packed, n, rank, world)
        assert local_n == n // world
        parts.append(c_oracle.decode_fp16(shard, local_n))
    np.testing.assert_array_equal(np.concatenate(parts, axis=0).view(np.uint16), full.view(np.uint16))
    with pytest.raises(ValueError):
        shard_columns(synthetic_sage(k, 40, seed=0), 40, 0, 2)


@pytest.mark.parametrize("world", [2, 4])
def test_row_shards_recombine(world):
    k, n = 1024, 48
    packed = synthetic_sage(k, n, seed=2)
    packed["permutation"] = block_permutation(k, 4, seed=5)
    full = c_oracle.decode_fp16(packed, n)  # original channel order
    per = k // world
    for rank in range(world):
        shard = shard_rows(packed, rank, world)
        local = c_oracle.decode_fp16(shard, n)  # [n, k/world], the rank's own channel order
        np.testing.assert_array_equal(local.view(np.uint16), full[:, rank * per : (rank + 1) * per].view(np.uint16))
    mixed = synthetic_sage(k, n, seed=2)  # a global permutation cannot be row-sharded
    with pytest.raises(ValueError):
        shard_rows(mixed, 0, world)
    x = torch.arange(2 * k).reshape(2, k)
    assert torch.equal(row_parallel_input(x, 1, world), x[:, per : 2 * per])
    table = torch.arange(64 * 8).reshape(64, 8)
    assert torch.equal(shard_vocab(table, 1, 4), table[16:32])


def test_output_rows_reorder_and_fold_keep_the_mlp():
    """A reference-style GLOBAL permutation on down_proj folded into gate/up's row order: the
    intermediate activations are the same values born in down_proj's quantised order, the MLP
    output is unchanged (FP32 sums in another order) and down_proj needs no gather."""
    hidden, inter = 256, 768
    gate, up = synthetic_sage(hidden, inter, seed=1), synthetic_sage(hidden, inter, seed=2)
    down = synthetic_sage(inter, hidden, seed=3)  # permutation: a global randperm of `inter`
    assert down["permutation"].numel() == inter
    order = torch.randperm(inter, generator=torch.Generator().manual_seed(0))
    moved = permute_output_rows(gate, inter, order)
    np.testing.assert_array_equal(c_oracle.decode_fp16(moved, inter).view(np.uint16),
                                  c_oracle.decode_fp16(gate, inter)[order.numpy()].view(np.uint16))
    x = torch.randn(2, hidden, generator=torch.Generator().manual_seed(5), dtype=torch.float16)

    def mlp(gate_p, up_p, down_p):
        g = torch.from_numpy(c_oracle.linear_fp32(x, gate_p, inter)).half()
        u = torch.from_numpy(c_oracle.linear_fp32(x, up_p, inter)).half()
        act = torch.nn.functional.silu(g.float()).half() * u
        return c_oracle.linear_fp32(act, down_p, hidden), act

    want, act = mlp(gate, up, down)
    (gate_f, up_f), down_f = fold_input_permutation([(gate, inter), (up, inter)], down)
    assert down_f["permutation"].numel() == 0
    got, act_f = mlp(gate_f, up_f, down_f)
    assert torch.equal(act_f, act[:, down["permutation"].long()])  # the intermediate is born in quantised order
    assert np.abs(got - want).max() <= 1e-5 * np.abs(want).max()
    # and a contiguous K split of the folded down_proj lines up with the column split of gate/up
    for world in (2, 3):
        total = np.zeros_like(want)
        for rank in range(world):
            (gate_r, n_r), (up_r, _) = shard_columns(gate_f, inter, rank, world), shard_columns(up_f, inter, rank, world)
            g = torch.from_numpy(c_oracle.linear_fp32(x, gate_r, n_r)).half()
            u = torch.from_numpy(c_oracle.linear_fp32(x, up_r, n_r)).half()
            local_act = torch.nn.functional.silu(g.float()).half() * u
            total += c_oracle.linear_fp32(local_act, shard_rows(down_f, rank, world), hidden)
        assert np.abs(total - want).max() <= 1e-5 * np.abs(want).max()


def test_global_permutation_row_shards_gather_from_the_full_row():
    k, n = 1024, 48
    packed = synthetic_sage(k, n, seed=2)  # a global permutation
    x = torch.randn(3, k, generator=torch.Generator().manual_seed(1), dtype=torch.float16)
    want = c_oracle.linear_fp32(x, packed, n)
    for world in (2, 4):
        total = np.zeros_like(want)
        for rank in range(world):
            shard, index = shard_rows_global(packed, rank, world)
            assert shard["permutation"].numel() == 0 and index.numel() == k // world
            total += c_oracle.linear_fp32(x[:, index].contiguous(), shard, n)
        assert np.abs(total - want).max() <= 1e-5 * np.abs(want).max()


def _worker(rank, world, path, k, n, results):
    dist.init_process_group("gloo", init_method=f"file://{path}", rank=rank, world_size=world)
    try:
        x = torch.randn(3, k, generator=torch.Generator().manual_seed(9), dtype=torch.float16)
        # row parallel: partial products summed with an all-reduce
        packed = synthetic_sage(k, n, seed=4)
        packed["permutation"] = block_permutation(k, 4, seed=6)
        want = torch.from_numpy(c_oracle.linear_fp32(x, packed, n))
        shard = shard_rows(packed, rank, world)
        partial = torch.from_numpy(c_oracle.linear_fp32(row_parallel_input(x, rank, world), shard, n))
        dist.all_reduce(partial)
        row_error = ((partial - want).norm() / want.norm()).item()
        # column parallel: every rank has the full input, outputs are concatenated
        shard, local_n = shard_columns(packed, n, rank, world)
        mine = torch.from_numpy(c_oracle.linear_fp32(x, shard, local_n))
        pieces = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(pieces, mine)
        column_error = ((torch.cat(pieces, dim=-1) - want).norm() / want.norm()).item()
        results.put((rank, row_error, column_error))
    finally:
        dist.destroy_process_group()


def test_two_rank_gloo_matches_unsharded():
    world, k, n = 2, 1024, 64
    context = mp.get_context("spawn")
    results = context.Queue()
    with tempfile.TemporaryDirectory() as folder:
        path = os.path.join(folder, "rendezvous")
        procs = [context.Process(target=_worker, args=(r, world, path, k, n, results)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(120)
            assert p.exitcode == 0
    seen = sorted(results.get(timeout=10) for _ in range(world))
    assert [r for r, _, _ in seen] == [0, 1]
    for _, row_error, column_error in seen:
        assert row_error < 1e-5 and column_error < 1e-6
