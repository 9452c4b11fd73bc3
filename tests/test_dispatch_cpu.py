"""Expert-parallel dispatch / combine on CPU: the slot bookkeeping of `dispatch_combine`
(owner selection, all-to-all, sort by expert, capacity, un-sort, combine, mixing) with a
stand-in expert function, on one process and on two gloo ranks that each own half of the
experts and their own tokens."""

import os
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from sage_b200.experts import dispatch_combine, route

HIDDEN, EXPERTS, TOP_K = 32, 8, 3


def expert_scale(expert: int) -> float:
    return 1.0 + 0.25 * expert  # expert e multiplies its input by this


def make_runner(first: int, local: int):
    def run(rows, block_experts):
        assert rows.shape[2] == HIDDEN and block_experts.shape[0] == rows.shape[0]
        assert bool(((block_experts == -1) | ((block_experts >= first) & (block_experts < first + local))).all())
        scales = torch.tensor([expert_scale(int(e)) if e >= 0 else float("nan") for e in block_experts])
        return rows * scales[:, None, None]  # (an unused block's rows turn into NaN: nobody may read them)

    return run


def expected(x, ids, weights):
    scales = torch.tensor([expert_scale(e) for e in range(EXPERTS)])
    return (x[:, None, :] * scales[ids.long()][..., None] * weights[..., None]).sum(dim=1)


def tokens_of(rank: int, count: int):
    gen = torch.Generator().manual_seed(100 + rank)
    x = torch.randn(count, HIDDEN, generator=gen)
    ids, weights = route(torch.randn(count, EXPERTS, generator=gen), TOP_K)
    return x, ids, weights


def test_one_rank_sorted_compute_matches_the_direct_sum():
    x, ids, weights = tokens_of(0, 11)
    got = dispatch_combine(x, ids, weights, make_runner(0, EXPERTS), first_expert=0, local_experts=EXPERTS)
    torch.testing.assert_close(got, expected(x, ids, weights), rtol=1e-6, atol=1e-6)


def test_crowded_experts_take_several_blocks():
    """Every token names the same three experts: nine rows each with blocks of four rows, so each
    of them owns three blocks and nothing is dropped."""
    x = torch.randn(9, HIDDEN)
    ids = torch.tensor([[0, 1, 2]] * 9, dtype=torch.int32)
    weights = torch.full((9, 3), 1 / 3)
    got = dispatch_combine(x, ids, weights, make_runner(0, EXPERTS), first_expert=0, local_experts=EXPERTS,
                           rows_per_block=4)
    torch.testing.assert_close(got, expected(x, ids, weights), rtol=1e-6, atol=1e-6)


def _worker(rank, world, path, results):
    dist.init_process_group("gloo", init_method=f"file://{path}", rank=rank, world_size=world)
    local = EXPERTS // world
    x, ids, weights = tokens_of(rank, 3 + rank)  # the ranks own different tokens (not even the same number...
    count = 3 + world                            # ...but the exchange needs equal slot counts: pad them)
    pad = count - x.shape[0]
    if pad:
        x = torch.cat((x, torch.zeros(pad, HIDDEN)))
        ids = torch.cat((ids, torch.zeros(pad, TOP_K, dtype=torch.int32)))
        weights = torch.cat((weights, torch.zeros(pad, TOP_K)))
    got = dispatch_combine(x, ids, weights, make_runner(rank * local, local), first_expert=rank * local,
                           local_experts=local, group=dist.group.WORLD, world=world, rows_per_block=4)
    results.put((rank, got, expected(x, ids, weights), 0))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_two_ranks_dispatch_and_combine(world):
    context = mp.get_context("spawn")
    results = context.Queue()
    with tempfile.TemporaryDirectory() as folder:
        procs = [context.Process(target=_worker, args=(rank, world, os.path.join(folder, "rendezvous"), results))
                 for rank in range(world)]
        for p in procs:
            p.start()
        gathered = [results.get(timeout=60) for _ in range(world)]
        for p in procs:
            p.join(60)
            assert p.exitcode == 0
    for rank, got, want, overflow in gathered:
        torch.testing.assert_close(got, want, rtol=1e-6, atol=1e-6)
        assert overflow == 0
