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

Expert parallelism: a rank constructs the module with its contiguous block of experts
(`first_expert`); slots routed to other ranks' experts contribute zeros, and the caller sums
the ranks' outputs (all-reduce) — every rank sees every token, so no dispatch is needed.
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
