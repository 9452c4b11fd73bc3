"""Packed mixture-of-experts MLP: the experts of one Qwen3-MoE layer as stacks of SAGE-packed
linears, driven by router output that stays on the GPU.

The reference has no packed MoE module: its inference wrappers are dense linears only and its
loader rejects every model type but `qwen3` (weight_vq/integrations/transformers.py:88-89);
experts exist only on its quantisation side, as per-expert names
`mlp.experts.{e}.{gate,up,down}_proj` (weight_vq/blockwise/artifacts.py:38-45).  `SAGEExperts`
keeps that naming's semantics — expert e is three independent packed linears — with the five
packed buffers of each projection stacked along a leading expert dimension, and follows the
routing arithmetic of Hugging Face `Qwen3MoeSparseMoeBlock` (softmax over all experts, top-k,
renormalise, weighted sum of the selected experts' SwiGLU MLPs).

Expert parallelism, two exchanges:
  * every rank sees every token (small batches): a rank constructs the module with its
    contiguous block of experts (`first_expert`); slots routed to other ranks' experts
    contribute zeros, and the caller sums the ranks' outputs (all-reduce) - no dispatch;
  * every rank owns its own tokens (`dispatch_combine`): each (token, expert) slot travels to
    the rank that owns the expert with `all_to_all_single`, the owner sorts what it received by
    expert, runs each local expert over its rows (`SAGEExperts.forward_blocks`), and a second
    `all_to_all_single` brings the outputs back.  All shapes are fixed (no host round trip), so
    the whole exchange is captured in the decode CUDA graph.
"""

from __future__ import annotations

import ctypes

import torch
from torch import nn

from . import _lib
from .ops import _workspace
from .synthetic import synthetic_sage_device

STACK_KEYS = ("packed_codes", "radius_codes", "radius_grid", "codebook", "permutation")


def synthetic_expert_stack(in_features: int, out_features: int, experts: int, seed: int, device,
                           *, direction_bits: int | None = None, first: int = 0) -> dict[str, torch.Tensor]:
    """`experts` synthetic packed linears of one shape and one bit split, stacked: the global
    experts first .. first+experts-1 (an expert's values depend on its global index only)."""
    bits = direction_bits if direction_bits is not None else 6 + seed % 3
    singles = [synthetic_sage_device(in_features, out_features, seed * 1009 + e, device, direction_bits=bits)
               for e in range(first, first + experts)]
    return {key: torch.stack([single[key] for single in singles]).contiguous() for key in STACK_KEYS}


def expert_slice(stack: dict[str, torch.Tensor], expert: int) -> dict[str, torch.Tensor]:
    """The five packed buffers of one expert (views), e.g. to build a `SAGELinear` from."""
    return {key: stack[key][expert] for key in STACK_KEYS}


def route(logits: torch.Tensor, top_k: int) -> tuple[torch.Tensor, torch.Tensor]:
    """Qwen3-MoE routing: softmax over all experts in FP32, top-k, renormalised weights.
    Returns (expert ids int32 [tokens, top_k], weights float32 [tokens, top_k])."""
    probabilities = torch.softmax(logits.float(), dim=-1)
    weights, ids = torch.topk(probabilities, top_k, dim=-1)
    weights = weights / weights.sum(dim=-1, keepdim=True)
    return ids.to(torch.int32), weights


ROWS_PER_EXPERT = 16  # rows one expert takes per step (the decode kernel's row limit)


def dispatch_combine(x: torch.Tensor, expert_ids: torch.Tensor, weights: torch.Tensor, run_blocks, *,
                     first_expert: int, local_experts: int, group=None, world: int = 1,
                     rows_per_block: int = ROWS_PER_EXPERT, state: dict | None = None,
                     use_kernels: bool | None = None) -> torch.Tensor:
    """Mixture-of-experts output of this rank's own tokens with the experts spread over `world`
    ranks: dispatch all-to-all, per-expert compute on the owners, combine all-to-all.

    x [tokens, hidden]; expert_ids int32 [tokens, top_k] (global ids); weights [tokens, top_k].
    What a rank receives is sorted by expert and cut into blocks of `rows_per_block` rows, every
    block belonging to one expert (an expert with many rows owns several blocks); the number of
    blocks is fixed at its worst case, local_experts + received / rows_per_block, so nothing
    depends on the routing and no slot is ever dropped.
    `run_blocks(rows, block_experts)`: rows [blocks, rows_per_block, hidden], block_experts int32
    [blocks] (global expert id, -1 for an unused block) -> [blocks, rows_per_block, hidden], row r
    of block b being that expert's MLP of that row (rows that carry no slot hold stale values and
    their outputs are never read).
    Returns [tokens, hidden] in x's dtype: sum_j weights[t, j] * expert_{ids[t, j]}(x[t]).
    On the GPU the receive side (plan, scatter into blocks, gather back, mix) runs as four kernels of
    this library; `use_kernels=False` keeps the tensor program below (the CPU path, and the
    reference the kernels are tested against)."""
    tokens, top_k = expert_ids.shape
    hidden = x.shape[1]
    slots = tokens * top_k
    device = x.device
    flat = expert_ids.reshape(slots).to(torch.int64)
    owner = torch.div(flat, local_experts, rounding_mode="floor")                      # rank that owns the slot's expert
    peers = torch.arange(world, device=device)[:, None]
    send_ids = torch.where(owner[None, :] == peers, flat[None, :], flat.new_full((), -1)).to(torch.int32).contiguous()
    received = world * slots
    kernels = (use_kernels is not False and x.is_cuda and x.dtype == torch.float16 and received <= 4096
               and local_experts <= 256 and hidden % 8 == 0)
    if use_kernels and not kernels:
        raise ValueError("the dispatch kernels take FP16 CUDA rows, at most 4096 received slots and 256 local experts")
    # (one GPU with the kernels: the scatter reads the tokens' rows directly, no per-slot copy)
    send_x = None if world == 1 and kernels else \
        x.repeat_interleave(top_k, dim=0)[None].expand(world, slots, hidden).contiguous()
    if world > 1:
        import torch.distributed as dist

        recv_x, recv_ids = torch.empty_like(send_x), torch.empty_like(send_ids)
        dist.all_to_all_single(recv_x, send_x, group=group)
        dist.all_to_all_single(recv_ids, send_ids, group=group)
    else:
        recv_x, recv_ids = send_x, send_ids
    blocks = local_experts + (received + rows_per_block - 1) // rows_per_block          # worst case, fixed
    if kernels:
        # on the GPU the plan, the scatter into blocks, the gather back and the mix are four launches
        return _dispatch_combine_kernels(x, recv_x if world > 1 else None, recv_ids, weights, run_blocks, tokens, top_k,
                                         hidden, received, blocks, first_expert, local_experts, rows_per_block,
                                         group, world, state)
    local = recv_ids.reshape(received).to(torch.int64) - first_expert
    key = torch.where(recv_ids.reshape(received) >= 0, local, local.new_full((), local_experts))  # empty slots sort last
    order = torch.argsort(key, stable=True)
    sorted_key = key[order]
    first_index = torch.searchsorted(sorted_key, torch.arange(local_experts + 1, device=device))
    counts = first_index[1:] - first_index[:-1]                                         # rows per local expert
    expert_blocks = torch.div(counts + rows_per_block - 1, rows_per_block, rounding_mode="floor")
    block_start = torch.cumsum(expert_blocks, 0) - expert_blocks                        # first block of each expert
    live = sorted_key < local_experts
    safe_key = torch.where(live, sorted_key, torch.zeros_like(sorted_key))
    position = torch.arange(received, device=device) - first_index[safe_key]
    block = block_start[safe_key] + torch.div(position, rows_per_block, rounding_mode="floor")
    dump = blocks * rows_per_block                                                      # a row nobody reads
    target = torch.where(live, block * rows_per_block + position % rows_per_block, position.new_full((), dump))
    # which expert each block serves: the blocks' first rows say so; the rest stay -1
    block_experts = torch.full((blocks + 1,), -1, dtype=torch.int32, device=device)
    heads = live & (position % rows_per_block == 0)
    block_experts.index_copy_(0, torch.where(heads, block, block.new_full((), blocks)),
                              torch.where(heads, sorted_key + first_expert, sorted_key.new_full((), -1)).to(torch.int32))
    if state is None:
        state = {}
    rows = state.get("rows")
    if rows is None or rows.shape != (dump + 1, hidden) or rows.device != device or rows.dtype != x.dtype:
        rows = state["rows"] = torch.zeros(dump + 1, hidden, dtype=x.dtype, device=device)
    rows.index_copy_(0, target, recv_x.reshape(received, hidden)[order])
    outputs = run_blocks(rows[:dump].view(blocks, rows_per_block, hidden), block_experts[:blocks])
    padded = torch.cat((outputs.reshape(dump, hidden), outputs.new_zeros(1, hidden)))
    back = torch.empty(received, hidden, dtype=x.dtype, device=device)
    back.index_copy_(0, order, padded[target])                                          # received order again
    back = back.view(world, slots, hidden)
    if world > 1:
        returned = torch.empty_like(back)
        dist.all_to_all_single(returned, back.contiguous(), group=group)
    else:
        returned = back
    slot_outputs = returned.sum(dim=0) if world > 1 else returned[0]                    # one block holds the value, the rest zeros
    mixed = (slot_outputs.view(tokens, top_k, hidden).float() * weights.to(torch.float32)[..., None]).sum(dim=1)
    return mixed.to(x.dtype)


def _dispatch_combine_kernels(x, recv_x, recv_ids, weights, run_blocks, tokens, top_k, hidden, received, blocks,
                              first_expert, local_experts, rows_per_block, group, world, state):
    """The receive side of `dispatch_combine` with this library's kernels (the same layout as the
    tensor program above: slots of an expert in received order, blocks in expert order)."""
    lib = _lib.load()
    device = x.device
    dump = blocks * rows_per_block
    if state is None:
        state = {}
    rows = state.get("rows")
    if rows is None or rows.shape != (dump + 1, hidden) or rows.device != device or rows.dtype != x.dtype:
        rows = state["rows"] = torch.zeros(dump + 1, hidden, dtype=x.dtype, device=device)
    target = torch.empty(received, dtype=torch.int32, device=device)
    block_experts = torch.empty(blocks, dtype=torch.int32, device=device)
    ids = recv_ids.reshape(received).contiguous()
    source = x.contiguous() if recv_x is None else recv_x.reshape(received, hidden)
    with torch.cuda.device(device):
        stream = torch.cuda.current_stream(device).cuda_stream

        def check(status, what):
            if status:
                raise RuntimeError(f"sage_b200: {what} failed with status {status}")

        check(lib.sageb200_glue_dispatch_plan(ids.data_ptr(), target.data_ptr(), block_experts.data_ptr(), received,
                                              first_expert, local_experts, rows_per_block, blocks, stream), "dispatch_plan")
        check(lib.sageb200_glue_dispatch_rows(source.data_ptr(), target.data_ptr(), rows.data_ptr(), received, hidden,
                                              dump, top_k if recv_x is None else 1, stream), "dispatch_rows")
        outputs = run_blocks(rows[:dump].view(blocks, rows_per_block, hidden), block_experts).contiguous()
        back = torch.empty(received, hidden, dtype=x.dtype, device=device)
        check(lib.sageb200_glue_combine_rows(outputs.data_ptr(), target.data_ptr(), back.data_ptr(), received, hidden,
                                             dump, stream), "combine_rows")
        if world > 1:
            import torch.distributed as dist

            returned = torch.empty_like(back)
            dist.all_to_all_single(returned, back, group=group)
            slot_outputs = returned.view(world, tokens * top_k, hidden).sum(dim=0)  # one rank holds the value, the rest zeros
        else:
            slot_outputs = back
        mixed = torch.empty(tokens, hidden, dtype=x.dtype, device=device)
        check(lib.sageb200_glue_moe_mix(slot_outputs.data_ptr(), weights.to(torch.float32).contiguous().data_ptr(),
                                        mixed.data_ptr(), tokens, hidden, top_k, stream), "moe_mix")
    return mixed


class SAGEExperts(nn.Module):
    """gate/up/down stacks of the experts [first_expert, first_expert + experts) of one layer."""

    def __init__(self, gate: dict, up: dict, down: dict, *, first_expert: int = 0):
        super().__init__()
        for prefix, stack in (("gate", gate), ("up", up), ("down", down)):
            for key in STACK_KEYS:
                self.register_buffer(f"{prefix}_{key}", stack[key])
        self.first_expert = first_expert
        self.experts = gate["packed_codes"].shape[0]
        self.hidden = gate["packed_codes"].shape[2] * 128
        self.intermediate = down["packed_codes"].shape[2] * 128

    def _stack(self, prefix: str, n: int, k: int) -> _lib.ExpertStack:
        get = lambda key: getattr(self, f"{prefix}_{key}")  # noqa: E731
        perm = get("permutation")
        return _lib.ExpertStack(
            get("packed_codes").data_ptr(), get("radius_codes").data_ptr(), get("radius_grid").data_ptr(),
            get("codebook").data_ptr(), perm.data_ptr() if perm.numel() else None, self.experts,
            self.first_expert, n, k, get("codebook").shape[2],
        )

    def _run(self, x: torch.Tensor, stride: int, stacks, outputs, ids: torch.Tensor, slots: int):
        lib = _lib.load()
        array = (_lib.ExpertStack * len(stacks))(*stacks)
        ys = (ctypes.c_void_p * len(outputs))(*[out.data_ptr() for out in outputs])
        stream = torch.cuda.current_stream(x.device).cuda_stream
        need = lib.sageb200_experts_workspace_bytes(array, len(stacks), slots)
        workspace = _workspace(x.device, stream, need) if need else None
        _lib.check(lib.sageb200_experts(
            x.data_ptr(), stride, array, ys, len(stacks), ids.data_ptr(), slots,
            workspace.data_ptr() if workspace is not None else None,
            workspace.numel() if workspace is not None else 0, stream))

    def forward_blocks(self, rows: torch.Tensor, block_experts: torch.Tensor) -> torch.Tensor:
        """rows FP16 [blocks, r <= 16, hidden], block_experts int32 [blocks] (global expert ids on the
        GPU, -1 = unused block): the SwiGLU MLP of each block's expert over the block's rows
        (gate and up, SwiGLU, down), the expert picked on the device."""
        blocks, count, hidden = rows.shape
        lib = _lib.load()
        half = dict(dtype=torch.float16, device=rows.device)
        gate = torch.zeros(blocks, count, self.intermediate, **half)
        up = torch.zeros(blocks, count, self.intermediate, **half)
        down = torch.zeros(blocks, count, self.hidden, **half)
        ids = block_experts.to(torch.int32).contiguous()

        def run(x, stacks, outputs):
            array = (_lib.ExpertStack * len(stacks))(*stacks)
            ys = (ctypes.c_void_p * len(outputs))(*[out.data_ptr() for out in outputs])
            stream = torch.cuda.current_stream(x.device).cuda_stream
            need = lib.sageb200_expert_blocks_workspace_bytes(array, len(stacks), count)
            workspace = _workspace(x.device, stream, need) if need else None
            _lib.check(lib.sageb200_expert_blocks(
                x.data_ptr(), array, ys, len(stacks), ids.data_ptr(), blocks, count,
                workspace.data_ptr() if workspace is not None else None,
                workspace.numel() if workspace is not None else 0, stream))

        with torch.cuda.device(rows.device):
            stream = torch.cuda.current_stream(rows.device).cuda_stream
            run(rows.contiguous(), [self._stack("gate", self.intermediate, self.hidden),
                                    self._stack("up", self.intermediate, self.hidden)], [gate, up])
            act = torch.empty_like(gate)
            status = lib.sageb200_glue_swiglu(gate.data_ptr(), up.data_ptr(), act.data_ptr(), gate.numel(), stream)
            if status:
                raise RuntimeError(f"sage_b200: swiglu failed with status {status}")
            run(act, [self._stack("down", self.hidden, self.intermediate)], [down])
        return down

    def forward(self, x: torch.Tensor, expert_ids: torch.Tensor, weights: torch.Tensor, *,
                foreign_experts: bool = True) -> torch.Tensor:
        """x FP16 [tokens, hidden]; expert_ids int32 [tokens, top_k]; weights [tokens, top_k].
        Returns this rank's experts' share of the MoE output, FP16 [tokens, hidden].
        `foreign_experts=False` promises that every id belongs to this rank (no expert
        parallelism), which saves zero-filling the slot buffers."""
        tokens, top_k = expert_ids.shape
        slots = tokens * top_k
        ids = expert_ids.reshape(-1).contiguous()
        lib = _lib.load()
        buffer = torch.zeros if foreign_experts else torch.empty
        with torch.cuda.device(x.device):
            stream = torch.cuda.current_stream(x.device).cuda_stream
            rows = x.contiguous() if tokens == 1 else x.repeat_interleave(top_k, dim=0).contiguous()
            gate = buffer(slots, self.intermediate, dtype=torch.float16, device=x.device)
            up = buffer(slots, self.intermediate, dtype=torch.float16, device=x.device)
            self._run(rows, 0 if tokens == 1 else self.hidden,
                      [self._stack("gate", self.intermediate, self.hidden),
                       self._stack("up", self.intermediate, self.hidden)], [gate, up], ids, slots)
            act = torch.empty_like(gate)
            status = lib.sageb200_glue_swiglu(gate.data_ptr(), up.data_ptr(), act.data_ptr(), gate.numel(), stream)
            if status:
                raise RuntimeError(f"sage_b200: swiglu failed with status {status}")
            down = buffer(slots, self.hidden, dtype=torch.float16, device=x.device)
            self._run(act, self.intermediate, [self._stack("down", self.hidden, self.intermediate)],
                      [down], ids, slots)
            mixed = torch.empty(tokens, self.hidden, dtype=torch.float16, device=x.device)
            weights = weights.to(torch.float32).contiguous()
            status = lib.sageb200_glue_moe_mix(down.data_ptr(), weights.data_ptr(), mixed.data_ptr(), tokens,
                                               self.hidden, top_k, stream)
            if status:
                raise RuntimeError(f"sage_b200: moe_mix failed with status {status}")
        return mixed
