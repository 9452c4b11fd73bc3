"""Random-initialised Qwen3 decoder whose linears are SAGE-packed, for decode benchmarks
and greedy-token parity.

The reference runs packed checkpoints inside Hugging Face `transformers` Qwen3
(weight_vq/integrations/transformers.py:83-164) and measures them with
benchmarks/model.py:43-133: StaticCache, one model call per generated token, the token kept
on the GPU.  This module is the same computation with the model glue written against the
decode kernels of libsage_b200 (include/sage_b200_decode.h): every step of a decode iteration
is enqueued on one stream without host synchronisation, so the iteration is captured once in
a CUDA graph and replayed per token.

`linear="sage"` runs the packed kernels; `linear="dense"` replaces every packed linear by an
FP16 `torch.nn.functional.linear` on the kernel-dequantised weight (the greedy-token oracle
the reference uses at tests/inference/test_hf_cuda.py:30-42), everything else identical.
"""

from __future__ import annotations

import ctypes
import dataclasses
import math

import torch

from . import _lib
from .ops import sage_dequantize, sage_forward_scratch, sage_grouped
from .experts import SAGEExperts, dispatch_combine, expert_slice, route, synthetic_expert_stack
from .parallel import (block_permutation, fold_input_permutation, shard_columns, shard_rows, shard_rows_global,
                       shard_vocab)
from .synthetic import linear_algorithmic_bytes, synthetic_sage_device


@dataclasses.dataclass(frozen=True)
class Qwen3Config:
    layers: int
    hidden: int
    heads: int
    kv_heads: int
    intermediate: int
    vocab: int = 151936
    head_dim: int = 128
    eps: float = 1e-6
    rope_theta: float = 1e6
    name: str = "qwen3"
    experts: int = 0           # > 0: mixture-of-experts MLP (Qwen3-MoE)
    top_k: int = 0
    moe_intermediate: int = 0


QWEN3_4B = Qwen3Config(layers=36, hidden=2560, heads=32, kv_heads=8, intermediate=9728, name="Qwen3-4B")
QWEN3_30B_A3B = Qwen3Config(layers=48, hidden=2048, heads=32, kv_heads=4, intermediate=6144, experts=128,
                            top_k=8, moe_intermediate=768, name="Qwen3-30B-A3B")
QWEN3_32B = Qwen3Config(layers=64, hidden=5120, heads=64, kv_heads=8, intermediate=25600, name="Qwen3-32B")


def _vp(tensor: torch.Tensor | None):
    return ctypes.c_void_p(tensor.data_ptr()) if tensor is not None else None


class PackedLinear:
    """One packed linear's buffers (and, for the oracle, its dense FP16 weight), optionally
    this rank's column- or row-parallel shard of it."""

    def __init__(self, k: int, n: int, seed: int, device, dense: bool, *, kind: str | None = None,
                 rank: int = 0, world: int = 1, perm_blocks: int = 1, packed: dict | None = None):
        """`packed`: this rank's buffers ready-made (k, n are then the shard's sizes); otherwise a
        seeded synthetic matrix is drawn and, under tensor parallelism, sharded by `kind`."""
        if packed is None:
            packed = synthetic_sage_device(k, n, seed, device, permuted=True)
            if kind == "row" and perm_blocks > 1:
                # row-parallel linears gather inside each rank's slice of the activations
                packed["permutation"] = block_permutation(k, perm_blocks, seed, device)
            if world > 1 and kind == "col":
                packed, n = shard_columns(packed, n, rank, world)
            elif world > 1 and kind == "row":
                packed = shard_rows(packed, rank, world)
                k //= world
        self.k, self.n = k, n
        self.entries = packed["codebook"].shape[1]
        self.bytes = linear_algorithmic_bytes(1, n, k, self.entries, packed["permutation"].numel() > 0)
        if dense:
            self.weight = sage_dequantize(
                packed["packed_codes"], packed["radius_codes"], packed["radius_grid"],
                packed["codebook"], packed["permutation"], n,
            )
            self.packed = None
        else:
            self.weight = None
            self.packed = packed

    def problem(self, x: torch.Tensor):
        p = self.packed
        return (x, p["packed_codes"], p["radius_codes"], p["radius_grid"], p["codebook"], p["permutation"])


class PackedQwen3:
    """Batch-`batch` greedy decoder with a static KV cache of `max_seq` positions."""

    def __init__(self, config: Qwen3Config, device, *, seed: int = 0, max_seq: int = 2560,
                 batch: int = 1, linear: str = "sage", max_new: int = 512, tp_group=None,
                 perm_blocks: int = 1, ep_group=None, ep_mode: str = "all_reduce",
                 collective: str = "peer"):
        """`tp_group`: a torch.distributed process group for tensor parallelism (q/k/v/gate/up
        column-parallel, o/down row-parallel with an all-reduce, vocabulary-parallel lm_head
        with an all-gather); every rank must pass the same seed.  `perm_blocks`: o/down use
        a block permutation with this many blocks (a multiple of the group size); 0 keeps the
        GLOBAL permutations an exported checkpoint has: down_proj's is folded into the row order
        of gate/up at load time, o_proj's is applied to the all-gathered attention output.
        `ep_group`: process group for expert parallelism of a mixture-of-experts config: each
        rank keeps experts/world contiguous experts.  `ep_mode` "all_reduce": every rank decodes
        the same `batch` sequences (attention and router replicated) and the ranks' expert outputs
        are summed with an all-reduce.  "all_to_all": every rank decodes its OWN `batch` sequences
        (data-parallel attention); each (token, expert) slot travels to the expert's owner with
        `all_to_all_single`, each local expert runs once over its rows, and a second all-to-all
        returns the outputs.  The same sorted per-expert compute serves one GPU when more than 16
        sequences decode together.
        `collective`: how the decode step's all-reduces run: "peer" = this library's one-kernel
        all-reduce over the peers' memory (sage_b200/peer.py; the GPUs of one node), "nccl" =
        `torch.distributed.all_reduce`.  Tensors larger than a decode step's (the prompt pass) always
        take NCCL."""
        if collective not in ("peer", "nccl"):
            raise ValueError("collective must be 'peer' or 'nccl'")
        if linear not in ("sage", "dense"):
            raise ValueError("linear must be 'sage' or 'dense'")
        if batch < 1 or batch > 64:
            raise ValueError("batch must be 1..64")
        if ep_mode not in ("all_reduce", "all_to_all"):
            raise ValueError("ep_mode must be 'all_reduce' or 'all_to_all'")
        self.config, self.device, self.batch, self.max_seq = config, torch.device(device), batch, max_seq
        self.dense = linear == "dense"
        self.tp_group = tp_group
        if tp_group is not None:
            import torch.distributed as dist

            self.tp_world, self.tp_rank = dist.get_world_size(tp_group), dist.get_rank(tp_group)
        else:
            self.tp_world, self.tp_rank = 1, 0
        world, rank = self.tp_world, self.tp_rank
        self.ep_group = ep_group
        if ep_group is not None:
            import torch.distributed as dist

            self.ep_world, self.ep_rank = dist.get_world_size(ep_group), dist.get_rank(ep_group)
        else:
            self.ep_world, self.ep_rank = 1, 0
        # (token, expert) slots sorted by expert and each expert run once over its rows: the
        # all-to-all exchange, and any mixture-of-experts batch beyond one grouped launch
        self.ep_dispatch = bool(config.experts) and (ep_mode == "all_to_all" or batch > 16)
        if self.ep_dispatch and ep_group is not None and ep_mode != "all_to_all":
            raise ValueError("more than 16 sequences under expert parallelism need ep_mode='all_to_all'")
        if config.experts and (config.experts % self.ep_world or world != 1):
            raise ValueError("experts must divide by the EP size; MoE configs do not combine with TP here")
        if config.heads % world or config.kv_heads % world or config.intermediate % (128 * world) or config.vocab % world:
            raise ValueError("heads, kv heads, intermediate/128 and vocabulary must divide by the TP size")
        if world > 1 and perm_blocks % world:
            raise ValueError("perm_blocks must be a multiple of the TP size")
        self.global_permutations = world > 1 and perm_blocks == 0
        # exchange buffers of the one-kernel all-reduce (row-parallel outputs, replicated-token
        # expert outputs): one decode step's [batch, hidden] rows
        self.peer = None
        self.prompt_chunk_rows = 0
        self.peer_error = ""
        reduce_group = tp_group if world > 1 else (ep_group if self.ep_world > 1 and ep_mode == "all_reduce" else None)
        if collective == "peer" and reduce_group is not None and not self.dense:
            from .peer import PeerExchange

            try:  # (all ranks succeed or all ranks raise, see PeerExchange)
                # (tensor parallelism also reduces chunks of prompt rows through the same exchange)
                self.prompt_chunk_rows = 512 if world > 1 else 0
                self.peer = PeerExchange(reduce_group, self.device,
                                         max(batch, self.prompt_chunk_rows) * config.hidden)
            except RuntimeError as error:  # the GPUs cannot map each other's memory here: NCCL serves
                self.peer = None
                self.peer_error = str(error)
        self.heads, self.kv_heads = config.heads // world, config.kv_heads // world
        self.lib = _lib.load()
        self.sm_count = torch.cuda.get_device_properties(self.device).multi_processor_count
        c = config
        gen = torch.Generator(device=self.device).manual_seed(seed)
        half = dict(device=self.device, dtype=torch.float16)
        self.embed = (torch.randn(c.vocab, c.hidden, generator=gen, device=self.device) * 0.02).half()
        # tied head, as in Qwen3-4B; under TP each rank keeps V/world rows of it
        self.lm_head = self.embed if world == 1 else shard_vocab(self.embed, rank, world)
        def norm_weight(width):  # random-init norms (around one) so the tests exercise them
            return (1.0 + 0.1 * torch.randn(width, generator=gen, device=self.device)).half()

        self.final_norm = norm_weight(c.hidden)
        self.layers = []
        q_out, kv_out = c.heads * c.head_dim, c.kv_heads * c.head_dim
        shapes = [("q", c.hidden, q_out, "col"), ("k", c.hidden, kv_out, "col"), ("v", c.hidden, kv_out, "col"),
                  ("o", q_out, c.hidden, "row"), ("gate", c.hidden, c.intermediate, "col"),
                  ("up", c.hidden, c.intermediate, "col"), ("down", c.intermediate, c.hidden, "row")]
        index = 0
        self.packed_bytes = 0
        for _ in range(c.layers):
            layer = {}
            drawn = {}
            for name, k, n, kind in shapes:
                if c.experts and name in ("gate", "up", "down"):
                    continue
                if self.global_permutations:  # the full matrices first: they are transformed together below
                    drawn[name] = synthetic_sage_device(k, n, seed * 100003 + index, self.device, permuted=True)
                else:
                    layer[name] = PackedLinear(k, n, seed * 100003 + index, self.device, self.dense, kind=kind,
                                               rank=rank, world=world, perm_blocks=perm_blocks)
                    self.packed_bytes += layer[name].bytes
                index += 1
            if self.global_permutations:
                if not c.experts:
                    (drawn["gate"], drawn["up"]), drawn["down"] = fold_input_permutation(
                        [(drawn["gate"], c.intermediate), (drawn["up"], c.intermediate)], drawn["down"])
                for name, k, n, kind in shapes:
                    if name not in drawn:
                        continue
                    if kind == "col":
                        shard, n = shard_columns(drawn[name], n, rank, world)
                    elif name == "o":
                        shard, layer["o_index"] = shard_rows_global(drawn[name], rank, world)
                        k //= world
                    else:
                        shard = shard_rows(drawn[name], rank, world)  # down: identity after the fold
                        k //= world
                    layer[name] = PackedLinear(k, n, 0, self.device, self.dense, packed=shard)
                    self.packed_bytes += layer[name].bytes
                del drawn
            if c.experts:
                local = c.experts // self.ep_world
                first = self.ep_rank * local
                base = (seed * 100003 + index) * 7919
                stacks = []
                for j, (k, n) in enumerate(((c.hidden, c.moe_intermediate), (c.hidden, c.moe_intermediate),
                                            (c.moe_intermediate, c.hidden))):
                    # every rank draws its own block of the same global experts
                    stacks.append(synthetic_expert_stack(k, n, local, base + j, self.device,
                                                         direction_bits=6 + (index + j) % 3, first=first))
                    self.packed_bytes += c.top_k * linear_algorithmic_bytes(1, n, k, 1 << (6 + (index + j) % 3), True)
                if self.dense:
                    from .ops import sage_dequantize as dq

                    layer["expert_weights"] = [
                        torch.stack([dq(*[expert_slice(stack, e)[key] for key in ("packed_codes", "radius_codes", "radius_grid", "codebook", "permutation")], n)
                                     for e in range(local)])
                        for stack, n in zip(stacks, (c.moe_intermediate, c.moe_intermediate, c.hidden))
                    ]
                else:
                    layer["experts"] = SAGEExperts(*stacks, first_expert=first)
                layer["first_expert"], layer["local_experts"] = first, local
                layer["router"] = (torch.randn(c.experts, c.hidden, generator=gen, device=self.device) * 0.5).half()
                index += 3
            layer["input_norm"] = norm_weight(c.hidden)
            layer["post_norm"] = norm_weight(c.hidden)
            layer["q_norm"] = norm_weight(c.head_dim)
            layer["k_norm"] = norm_weight(c.head_dim)
            layer["k_cache"] = torch.zeros(batch, self.kv_heads, max_seq, c.head_dim, **half)
            layer["v_cache"] = torch.zeros(batch, self.kv_heads, max_seq, c.head_dim, **half)
            # several sequences per step: the attention kernel writes its rows through the inverse of
            # o_proj's permutation, i.e. in o_proj's quantised channel order, and o_proj is then called
            # without a permutation (no staging launch in front of it)
            layer["o_inverse"] = None
            if batch > 1 and not self.dense and not self.global_permutations:
                perm = layer["o"].packed["permutation"]
                if perm.numel() == q_out // world:
                    inverse = torch.empty_like(perm)
                    inverse[perm.long()] = torch.arange(perm.numel(), dtype=perm.dtype, device=perm.device)
                    layer["o_inverse"] = inverse
            self.layers.append(layer)
        # rotary tables, computed in FP32 and rounded to FP16 as the HF module does
        inv_freq = 1.0 / (c.rope_theta ** (torch.arange(0, c.head_dim, 2, device=self.device).float() / c.head_dim))
        angles = torch.arange(max_seq, device=self.device).float()[:, None] * inv_freq[None, :]
        self.cos, self.sin = angles.cos().half().contiguous(), angles.sin().half().contiguous()
        # state
        self.tokens = torch.zeros(batch, dtype=torch.int64, device=self.device)
        self.positions = torch.zeros(batch, dtype=torch.int32, device=self.device)
        self.step_counter = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.log = torch.zeros(batch, max_new, dtype=torch.int64, device=self.device)
        self.max_new = max_new
        self.h = torch.zeros(batch, c.hidden, **half)
        self.h_other = torch.zeros(batch, c.hidden, **half)  # residual ping-pong for fused norms
        self.fuse = True
        self.scratch = None  # zero-filled scratch of the packed linears above 16 rows (see _packed_rows)
        self.retired_scratch = []
        self.x = torch.zeros(batch, c.hidden, **half)
        self.attn = torch.zeros(batch, q_out // world, **half)
        self.attn_all = torch.zeros(world, batch, q_out // world, **half) if self.global_permutations else None
        self.act = torch.zeros(batch, c.intermediate // world, **half)
        self.logits = torch.zeros(batch, c.vocab, **half)
        self.local_logits = torch.zeros(batch, c.vocab // world, **half) if world > 1 else self.logits
        self.gathered_logits = torch.zeros(world, batch, c.vocab // world, **half) if world > 1 else None
        self.splits = 16
        scratch = self.lib.sageb200_glue_attention_scratch_bytes(batch, self.heads, self.splits)
        self.attn_scratch = torch.zeros(scratch // 4, dtype=torch.float32, device=self.device)
        # single-launch attention and step tail (`fuse_glue`); the tail's arrival counter starts at zero
        self.fuse_glue = True
        # CTAs per cluster in the single-launch attention (each takes a share of the context): as many
        # as keep (sequences x kv heads x splits) within about one wave of SMs, 8 at most
        self.step_splits = 8
        while self.step_splits > 1 and batch * self.kv_heads * self.step_splits > self.sm_count:
            self.step_splits //= 2
        scratch = self.lib.sageb200_glue_lm_head_step_scratch_bytes(batch, self.sm_count)
        self.head_scratch = torch.zeros(scratch // 4, dtype=torch.float32, device=self.device)
        if c.experts:
            self.route_ids = torch.zeros(batch, c.top_k, dtype=torch.int32, device=self.device)
            self.route_weights = torch.zeros(batch, c.top_k, dtype=torch.float32, device=self.device)
        self.graph = None
        self.graph_no_head = None
        # what the expert-parallel exchange of a step is, for reports
        self.ep_collective = "nccl all_reduce of the ranks' expert outputs (every rank holds every token)"
        if self.peer is not None and self.ep_world > 1:
            self.ep_collective = ("one-kernel all-reduce of the ranks' expert outputs over peer memory "
                                  "(push over NVLink, epoch flags, rank-order sum; every rank holds every token)")
        self.tp_collective = ("one-kernel all-reduce over peer memory (row-parallel partial sums: push over NVLink, "
                              "epoch flags, rank-order sum) + nccl all_gather (logits)" if self.peer is not None
                              else "nccl all_reduce (row-parallel partial sums) + all_gather (logits)")
        self.collective_calls_per_step = c.layers if self.ep_world > 1 else 0
        if self.ep_dispatch and self.ep_world > 1:
            self.ep_collective = ("nccl all_to_all_single: dispatch of (token, expert) slots (rows and ids) to the "
                                  "experts' owners, combine of their outputs (every rank owns its own tokens)")
            self.collective_calls_per_step = 3 * c.layers
        self._dispatch_state = {}
        self.ep_rows_per_block = 8  # rows of one expert block in the sorted expert compute (one MMA column block)
        # The whole token as one persistent kernel (`sageb200_mega_step`).  Prepared when the model
        # fits it; `use_mega` selects it for the decode step before `capture()`.  It is off by
        # default: as measured on B200 the per-launch path is still the faster one.
        self.mega = None
        self.use_mega = False
        if not self.dense and batch == 1 and world == 1 and self.ep_world == 1 and not c.experts:
            self._prepare_mega()
            self.use_mega = False

    # ------------------------------------------------------------------ the one-kernel decode step

    def _prepare_mega(self):
        """Describe the model to `sageb200_mega_prepare`; leaves `use_mega` False when the
        model does not fit that kernel (the per-launch path then serves every step)."""
        c, lib = self.config, self.lib
        model = _lib.MegaModel(c.layers, c.hidden, c.heads, c.kv_heads, c.head_dim, c.intermediate, c.vocab,
                               self.max_seq, c.eps, self.embed.data_ptr(), self.lm_head.data_ptr(),
                               self.final_norm.data_ptr(), self.cos.data_ptr(), self.sin.data_ptr())
        nbytes = lib.sageb200_mega_workspace_bytes(ctypes.byref(model), self.sm_count)
        if nbytes == 0:
            return
        layers = (_lib.MegaLayer * c.layers)()
        for index, layer in enumerate(self.layers):
            entry = layers[index]
            for name in ("q", "k", "v", "o", "gate", "up", "down"):
                linear, p = layer[name], layer[name].packed
                perm = p["permutation"]
                if perm.numel() and perm.data_ptr() % 16:
                    return
                setattr(entry, name, _lib.MegaLinear(
                    p["packed_codes"].data_ptr(), p["radius_codes"].data_ptr(), p["radius_grid"].data_ptr(),
                    p["codebook"].data_ptr(), perm.data_ptr() if perm.numel() else None, linear.n, linear.k,
                    linear.entries))
            for name in ("input_norm", "post_norm", "q_norm", "k_norm", "k_cache", "v_cache"):
                setattr(entry, name, layer[name].data_ptr())
        workspace = torch.zeros(nbytes, dtype=torch.uint8, device=self.device)
        with torch.cuda.device(self.device):
            status = lib.sageb200_mega_prepare(ctypes.byref(model), layers, _vp(workspace), nbytes, self._stream())
        self._check(status, "mega_prepare")
        self.mega = (model, workspace)

    def _mega_step(self):
        model, workspace = self.mega
        self._check(self.lib.sageb200_mega_step(
            ctypes.byref(model), _vp(workspace), _vp(self.tokens), _vp(self.positions), _vp(self.log),
            _vp(self.step_counter), _vp(self.logits), self.max_new, self._stream()), "mega_step")

    # ------------------------------------------------------------------ pieces

    def _stream(self):
        return ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)

    def _check(self, status: int, what: str):
        if status:
            raise RuntimeError(f"sage_b200 decode glue: {what} failed with status {status}")

    def _linears(self, layer, names, x, activation=None):
        if self.dense:
            return [torch.nn.functional.linear(x, layer[name].weight) for name in names]
        if self.batch > 16:  # beyond a grouped launch: one call per linear (decode kernel in two
            return self._rows_linears(layer, names, x)  # passes up to 32 rows, tensor-core GEMM above)
        return sage_grouped([layer[name].problem(x) for name in names], [layer[name].n for name in names],
                            activation)

    def _norm_linears(self, layer, names, delta, weight):
        """x = rmsnorm(h + delta) * weight, h += delta, then the packed linears `names` on x.
        Packed path: one launch (the norm runs inside the decode kernel's activation staging
        and the new residual goes to the other of two residual buffers).  Dense oracle: the
        stand-alone norm kernel, then torch matmuls."""
        c, lib, b = self.config, self.lib, self.batch
        if self.dense or not self.fuse or b > 16:
            self._check(lib.sageb200_glue_add_rmsnorm(_vp(self.h), _vp(delta), _vp(weight), _vp(self.x), b,
                                                      c.hidden, c.eps, self._stream()), "add_rmsnorm")
            return self._linears(layer, names, self.x)
        out = self._linears(layer, names, self.h, (1, c.eps, self.h, delta, weight, self.h_other))
        self.h, self.h_other = self.h_other, self.h
        return out

    def _all_reduce(self, tensor):
        """Sum the row-parallel partial outputs over the tensor-parallel group: one kernel over
        the peers' memory for a decode step's rows, NCCL for anything larger."""
        if self.tp_world > 1:
            if self.peer is not None and self.peer.fits(tensor):
                self.peer.all_reduce(tensor)
                return
            import torch.distributed as dist

            dist.all_reduce(tensor, group=self.tp_group)

    def _layer(self, layer, delta):
        """One decoder layer; `delta` is the previous layer's MLP output still to be added to
        the residual stream (None for the first layer).  Returns this layer's MLP output."""
        c, lib, b = self.config, self.lib, self.batch
        s = self._stream()
        q, k, v = self._norm_linears(layer, ("q", "k", "v"), delta, layer["input_norm"])
        if self.fuse_glue and layer["o_inverse"] is not None:
            self._check(lib.sageb200_glue_attention_step_permuted(
                _vp(q), _vp(k), _vp(v), _vp(layer["q_norm"]), _vp(layer["k_norm"]), _vp(self.cos), _vp(self.sin),
                _vp(self.positions), _vp(layer["k_cache"]), _vp(layer["v_cache"]), _vp(self.attn),
                _vp(layer["o_inverse"]), b, self.heads, self.kv_heads, c.head_dim, self.max_seq, self.step_splits,
                c.eps, s), "attention_step_permuted")
            return self._after_attention(layer, pregathered=True)
        if self.fuse_glue:
            self._check(lib.sageb200_glue_attention_step(
                _vp(q), _vp(k), _vp(v), _vp(layer["q_norm"]), _vp(layer["k_norm"]), _vp(self.cos), _vp(self.sin),
                _vp(self.positions), _vp(layer["k_cache"]), _vp(layer["v_cache"]), _vp(self.attn),
                b, self.heads, self.kv_heads, c.head_dim, self.max_seq, self.step_splits, c.eps, s),
                "attention_step")
            return self._after_attention(layer)
        self._check(lib.sageb200_glue_qk_norm_rope_cache(
            _vp(q), _vp(k), _vp(v), _vp(layer["q_norm"]), _vp(layer["k_norm"]), _vp(self.cos),
            _vp(self.sin), _vp(self.positions), _vp(layer["k_cache"]), _vp(layer["v_cache"]), b,
            self.heads, self.kv_heads, c.head_dim, self.max_seq, c.eps, s), "qk_norm_rope_cache")
        self._check(lib.sageb200_glue_attention_decode(
            _vp(q), _vp(layer["k_cache"]), _vp(layer["v_cache"]), _vp(self.positions), _vp(self.attn),
            _vp(self.attn_scratch), b, self.heads, self.kv_heads, c.head_dim, self.max_seq, self.splits, s),
            "attention_decode")
        return self._after_attention(layer)

    def _after_attention(self, layer, pregathered=False):
        c, lib, b = self.config, self.lib, self.batch
        s = self._stream()
        attn = self.attn
        if self.global_permutations:
            # o_proj's global permutation: every rank's heads gathered (a few KB), then this rank's
            # K slice picks its source channels out of the full row
            import torch.distributed as dist

            dist.all_gather_into_tensor(self.attn_all, self.attn, group=self.tp_group)
            attn = self.attn_all.permute(1, 0, 2).reshape(b, -1).index_select(-1, layer["o_index"])
        if pregathered:  # (the rows already lie in o_proj's quantised channel order)
            o = self._pregathered(layer["o"], attn)
        else:
            (o,) = self._linears(layer, ("o",), attn)
        self._all_reduce(o)
        if c.experts:
            return self._moe(layer, o)
        gate, up = self._norm_linears(layer, ("gate", "up"), o, layer["post_norm"])
        if self.dense or not self.fuse or b > 16:
            self._check(lib.sageb200_glue_swiglu(_vp(gate), _vp(up), _vp(self.act), gate.numel(), s), "swiglu")
            (down,) = self._linears(layer, ("down",), self.act)
        else:  # SwiGLU inside the down projection's activation staging
            (down,) = self._linears(layer, ("down",), self.act, (2, 0.0, gate, up, None, None))
        self._all_reduce(down)
        return down

    def _moe(self, layer, o):
        """Mixture-of-experts MLP: norm, FP16 router, top-k routing on the GPU, routed packed
        experts (this rank's block), all-reduce over the expert-parallel group."""
        c, lib, b = self.config, self.lib, self.batch
        if self.fuse_glue:  # norm + router + top-k in one launch (both the packed and the dense model)
            ids, weights = self.route_ids, self.route_weights
            self._check(lib.sageb200_glue_moe_route(
                _vp(self.h), _vp(o), _vp(layer["post_norm"]), _vp(layer["router"]), _vp(self.x), _vp(ids),
                _vp(weights), b, c.hidden, c.experts, c.top_k, c.eps, self._stream()), "moe_route")
        else:
            self._check(lib.sageb200_glue_add_rmsnorm(_vp(self.h), _vp(o), _vp(layer["post_norm"]), _vp(self.x), b,
                                                      c.hidden, c.eps, self._stream()), "add_rmsnorm")
            ids, weights = route(torch.nn.functional.linear(self.x, layer["router"]), c.top_k)
        if self.ep_dispatch:
            if self.dense:
                gate_w, up_w, down_w = layer["expert_weights"]
                first, count = layer["first_expert"], layer["local_experts"]

                def run_blocks(rows, block_experts):  # FP16 matmuls on the dequantised experts
                    index = (block_experts.long() - first).clamp(0, count - 1)
                    g = torch.bmm(rows, gate_w[index].transpose(1, 2))
                    u = torch.bmm(rows, up_w[index].transpose(1, 2))
                    act = torch.nn.functional.silu(g.float()).half() * u
                    return torch.bmm(act, down_w[index].transpose(1, 2))
            else:
                run_blocks = layer["experts"].forward_blocks
            return dispatch_combine(self.x, ids, weights, run_blocks, first_expert=layer["first_expert"],
                                    local_experts=layer["local_experts"], group=self.ep_group, world=self.ep_world,
                                    rows_per_block=self.ep_rows_per_block, state=self._dispatch_state)
        if self.dense:
            gate_w, up_w, down_w = layer["expert_weights"]
            local = ids.long() - layer["first_expert"]
            mine = (local >= 0) & (local < layer["local_experts"])
            index = local.clamp(0, layer["local_experts"] - 1)
            x = self.x[:, None, :, None]                                        # [b, 1, hidden, 1]
            g = torch.matmul(gate_w[index], x).squeeze(-1)                       # [b, top_k, inter]
            u = torch.matmul(up_w[index], x).squeeze(-1)
            act = torch.nn.functional.silu(g.float()).half() * u
            d = torch.matmul(down_w[index], act[..., None]).squeeze(-1)          # [b, top_k, hidden]
            out = (d.float() * (weights * mine)[..., None]).sum(dim=1).half()
        else:
            out = layer["experts"](self.x, ids, weights, foreign_experts=self.ep_world > 1)
        if self.ep_world > 1:
            if self.peer is not None and self.peer.fits(out):
                self.peer.all_reduce(out)
                return out
            import torch.distributed as dist

            dist.all_reduce(out, group=self.ep_group)
        return out

    def _body(self):
        c, lib, b = self.config, self.lib, self.batch
        s = self._stream()
        self._check(lib.sageb200_glue_embed(_vp(self.embed), _vp(self.tokens), _vp(self.h), b, c.hidden, c.vocab, s), "embed")
        delta = None
        for layer in self.layers:
            delta = self._layer(layer, delta)
        return delta

    def step(self, head: bool = True):
        """Enqueue one decode iteration for the tokens in `self.tokens` at `self.positions`."""
        c, lib, b = self.config, self.lib, self.batch
        if head and self.use_mega:
            self._mega_step()  # the whole token, lm_head and argmax included, in one kernel
            return
        delta = self._body()
        s = self._stream()
        if not head:
            self.positions.add_(1)
            return
        self._tail(self.h, delta)

    def _tail(self, residual, delta):
        """Final norm of residual + delta, lm_head, greedy argmax, token log and position advance."""
        c, lib, b = self.config, self.lib, self.batch
        s = self._stream()
        if self.fuse_glue and not self.dense and self.tp_world == 1 and b <= 16:
            self._check(lib.sageb200_glue_lm_head_step(
                _vp(self.lm_head), _vp(residual), _vp(delta), _vp(self.final_norm), _vp(self.x), _vp(self.logits),
                _vp(self.tokens), _vp(self.positions), _vp(self.log), _vp(self.step_counter),
                _vp(self.head_scratch), b, c.vocab, c.hidden, c.eps, self.max_new, self.sm_count, s),
                "lm_head_step")
            return
        self._check(lib.sageb200_glue_add_rmsnorm(_vp(residual), _vp(delta), _vp(self.final_norm),
                                                  _vp(self.x), b, c.hidden, c.eps, s), "final norm")
        local_vocab = c.vocab // self.tp_world
        if self.dense:
            torch.matmul(self.x, self.lm_head.T, out=self.local_logits)
        else:
            for first in range(0, b, 16):  # the head kernel takes up to 16 rows at a time
                rows = min(16, b - first)
                self._check(lib.sageb200_glue_lm_head(_vp(self.lm_head), _vp(self.x[first:]),
                                                      _vp(self.local_logits[first:]), rows, local_vocab, c.hidden,
                                                      self.sm_count, s), "lm_head")
        if self.tp_world > 1:
            import torch.distributed as dist

            dist.all_gather_into_tensor(self.gathered_logits, self.local_logits, group=self.tp_group)
            self.logits.view(b, self.tp_world, local_vocab).copy_(self.gathered_logits.permute(1, 0, 2))
        self._check(lib.sageb200_glue_argmax_advance(_vp(self.logits), _vp(self.tokens), _vp(self.positions),
                                                     _vp(self.log), _vp(self.step_counter), b, c.vocab,
                                                     self.max_new, s), "argmax")

    # ------------------------------------------------------------------ graphs and drivers

    def capture(self):
        """Capture the decode iteration (with and without the lm_head) in CUDA graphs.

        Warm-up and capture run on one stream owned by the model, so everything that is
        cached per stream (this library's scratch, cuBLAS workspaces of the dense oracle) is
        allocated by the eager warm-up and not inside a graph's private memory pool, which
        would go away with the graph while the cache still points at it."""
        saved = (self.tokens.clone(), self.positions.clone(), self.step_counter.clone(), self.log.clone())
        stream = torch.cuda.Stream(device=self.device)
        stream.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(stream):
            self.step(head=True)
            self.step(head=False)
        torch.cuda.current_stream(self.device).wait_stream(stream)
        torch.cuda.synchronize(self.device)
        self.graph, self.graph_no_head = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
        launches, glue = self.lib.sageb200_launch_count(), self.lib.sageb200_glue_launch_count()
        with torch.cuda.graph(self.graph, stream=stream):
            self.step(head=True)
        self.sage_launches_per_step = self.lib.sageb200_launch_count() - launches
        self.glue_launches_per_step = self.lib.sageb200_glue_launch_count() - glue
        with torch.cuda.graph(self.graph_no_head, stream=stream):
            self.step(head=False)
        self.tokens.copy_(saved[0])
        self.positions.copy_(saved[1])
        self.step_counter.copy_(saved[2])
        self.log.copy_(saved[3])
        torch.cuda.synchronize(self.device)

    def reset(self):
        self.positions.zero_()
        self.step_counter.zero_()
        self.log.zero_()

    def prefill(self, prompt: torch.Tensor, batched: bool | None = None):
        """Run `prompt` [batch, length] into the cache; after it, `self.tokens` holds the first
        generated token.  `batched` (the default on one GPU for a dense-MLP config): all
        prompt tokens go through each layer together - packed linears on the tensor-core GEMM
        path from 33 rows up, causal attention over the prompt.  Otherwise the prompt is fed
        one position at a time through the decode graph."""
        if self.graph is None:
            self.capture()
        if prompt.dim() != 2 or prompt.shape[0] != self.batch:
            raise ValueError("prompt must be [batch, length]")
        if prompt.shape[1] < 1 or prompt.shape[1] > self.max_seq:
            raise ValueError(f"prompt length {prompt.shape[1]} does not fit the cache of {self.max_seq} positions")
        if int(prompt.min()) < 0 or int(prompt.max()) >= self.config.vocab:
            raise ValueError("prompt token ids must lie in [0, vocab)")
        self.reset()
        prompt = prompt.to(self.device)
        length = prompt.shape[1]
        if batched is None:
            batched = (self.ep_world == 1 and not self.config.experts and length > 1
                       and self.batch * length <= 65535 and (self.tp_world == 1 or self._tp_prompt_ok()))
        if batched and self.tp_world > 1:
            return self._prefill_batched_tp(prompt)
        if batched:
            return self._prefill_batched(prompt)
        for i in range(length):
            self.tokens.copy_(prompt[:, i])
            (self.graph if i == length - 1 else self.graph_no_head).replay()

    def _tp_prompt_ok(self) -> bool:
        """Batched prompt rows under tensor parallelism need the one-kernel all-reduce (an eager NCCL
        collective after the decode graphs were captured is not an option here) and per-rank
        permutations (no all-gather of the attention output)."""
        return (self.peer is not None and self.prompt_chunk_rows > 0 and not self.global_permutations
                and not self.dense)

    def _prefill_batched_tp(self, prompt: torch.Tensor):
        """The prompt under tensor parallelism: all tokens but the last go through every layer in
        chunks of rows (column-parallel q/k/v/gate/up and row-parallel o/down on the tensor-core GEMM
        path, this rank's heads in the tensor-core attention, the row-parallel partial sums reduced by
        the one-kernel all-reduce over peer memory), which fills the KV cache; the last prompt token
        then takes the captured decode step, whose tail (vocabulary-parallel lm_head, all-gather of
        the logits, argmax) yields the first generated token."""
        if not self._tp_prompt_ok():
            raise ValueError("batched prompt rows under tensor parallelism need the peer all-reduce and block permutations")
        c, lib, b = self.config, self.lib, self.batch
        length = prompt.shape[1]
        half = dict(dtype=torch.float16, device=self.device)
        body = length - 1
        per_chunk = max(1, self.prompt_chunk_rows // b)  # tokens of every sequence per chunk
        with torch.cuda.device(self.device):
            s = self._stream()
            first = 0
            while first < body:
                count = min(per_chunk, body - first)
                rows = b * count  # row = sequence * count + token
                tokens = prompt[:, first:first + count].reshape(-1).to(torch.int64).contiguous()
                h = torch.empty(rows, c.hidden, **half)
                attn = torch.empty(rows, self.heads * c.head_dim, **half)
                self._check(lib.sageb200_glue_embed(_vp(self.embed), _vp(tokens), _vp(h), rows, c.hidden, c.vocab, s), "embed")
                delta = None
                for layer in self.layers:
                    q, k, v = self._norm_rows_linears(layer, ("q", "k", "v"), h, delta, layer["input_norm"], rows)
                    self._check(lib.sageb200_glue_prefill_qk_norm_rope_cache(
                        _vp(q), _vp(k), _vp(v), _vp(layer["q_norm"]), _vp(layer["k_norm"]), _vp(self.cos), _vp(self.sin),
                        _vp(self.positions), _vp(layer["k_cache"]), _vp(layer["v_cache"]), b, count, self.heads,
                        self.kv_heads, c.head_dim, self.max_seq, c.eps, s), "prefill_qk_norm_rope_cache")
                    self._check(lib.sageb200_glue_prefill_attention(
                        _vp(q), _vp(layer["k_cache"]), _vp(layer["v_cache"]), _vp(self.positions), _vp(attn), b, count,
                        self.heads, self.kv_heads, c.head_dim, self.max_seq, s), "prefill_attention")
                    (o,) = self._rows_linears(layer, ("o",), attn)
                    self.peer.all_reduce(o)
                    gate, up = self._norm_rows_linears(layer, ("gate", "up"), h, o, layer["post_norm"], rows)
                    delta = self._swiglu_rows_linear(layer, "down", gate, up)
                    self.peer.all_reduce(delta)
                self.positions.add_(count)
                first += count
            # the last prompt token: one captured decode step on top of the filled cache
            self.tokens.copy_(prompt[:, length - 1])
            self.graph.replay()

    def _packed_rows(self, linear, x, permutation):
        """One packed linear on rows `x`, with scratch memory the model owns (zero-filled, grown by the
        eager warm-up that precedes every capture), so that a captured step holds no temporary and
        no fill kernel per call."""
        p = linear.packed
        rows = x.numel() // x.shape[-1]
        if rows <= 16:  # (the grouped entry keeps its own scratch per stream)
            return sage_grouped([(x, p["packed_codes"], p["radius_codes"], p["radius_grid"], p["codebook"],
                                  permutation)], [linear.n])[0]
        nbytes = self.lib.sageb200_workspace_bytes(rows, linear.n, x.shape[-1])
        if self.scratch is None or self.scratch.numel() < nbytes:
            if self.scratch is not None:  # (a captured graph may still point at the smaller one)
                self.retired_scratch.append(self.scratch)
            self.scratch = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=self.device)
        return sage_forward_scratch(x, p["packed_codes"], p["radius_codes"], p["radius_grid"], p["codebook"],
                                    permutation, linear.n, self.scratch)

    def _grouped_row_blocks(self, linears, x, permutations):
        """17..32 rows: every linear as two row blocks of 9..16 rows, all blocks of all linears
        in ONE grouped launch of the decode kernel (and one staging launch for their permutations)
        instead of two launches and two staging launches per linear."""
        rows = x.shape[0]
        outs = [torch.empty(rows, linear.n, dtype=x.dtype, device=x.device) for linear in linears]
        problems, widths, targets = [], [], []
        for linear, permutation, out in zip(linears, permutations, outs):
            p = linear.packed
            half = (rows + 1) // 2  # (two blocks of the same kind: both above eight rows)
            for first in range(0, rows, half):
                block = slice(first, min(first + half, rows))
                problems.append((x[block], p["packed_codes"], p["radius_codes"], p["radius_grid"], p["codebook"],
                                 permutation))
                widths.append(linear.n)
                targets.append(out[block])
        sage_grouped(problems, widths, outputs=targets)
        return outs

    def _pregathered(self, linear, xq):
        """A packed linear on activations that already lie in its quantised channel order."""
        if xq.dim() == 2 and 16 < xq.shape[0] <= 32:
            return self._grouped_row_blocks([linear], xq, [linear.packed["permutation"][:0]])[0]
        return self._packed_rows(linear, xq, linear.packed["permutation"][:0])

    def _norm_rows_linears(self, layer, names, h, delta, weight, rows):
        """Prompt rows: h += delta, x = rmsnorm(h) * weight, then the packed linears `names` on x.  The
        norm kernel writes x once per linear in that linear's quantised channel order, so the
        linears need no gather pre-pass (dense oracle model, or a linear without a permutation: the
        plain norm kernel and the usual call)."""
        c, lib = self.config, self.lib
        s = self._stream()
        permutations = [] if self.dense else [layer[name].packed["permutation"] for name in names]
        if self.dense or len(names) > 4 or any(p.numel() != c.hidden or p.data_ptr() % 16 for p in permutations):
            x = torch.empty_like(h)
            self._check(lib.sageb200_glue_add_rmsnorm(_vp(h), _vp(delta), _vp(weight), _vp(x), rows, c.hidden, c.eps, s),
                        "add_rmsnorm")
            return self._rows_linears(layer, names, x)
        outs = [torch.empty_like(h) for _ in names]
        perm_array = (ctypes.c_void_p * len(names))(*[p.data_ptr() for p in permutations])
        out_array = (ctypes.c_void_p * len(names))(*[o.data_ptr() for o in outs])
        self._check(lib.sageb200_glue_add_rmsnorm_permuted(_vp(h), _vp(delta), _vp(weight), None, perm_array, out_array,
                                                           len(names), rows, c.hidden, c.eps, s), "add_rmsnorm_permuted")
        return [self._pregathered(layer[name], xq) for name, xq in zip(names, outs)]

    def _swiglu_rows_linear(self, layer, name, gate, up):
        """Prompt rows: the packed linear `name` on SwiGLU(gate, up), the activation written directly
        in the linear's quantised channel order where it has a permutation."""
        lib = self.lib
        s = self._stream()
        act = torch.empty_like(gate)
        permutation = None if self.dense else layer[name].packed["permutation"]
        k = gate.shape[-1]
        if permutation is None or permutation.numel() != k or permutation.data_ptr() % 16:
            self._check(lib.sageb200_glue_swiglu(_vp(gate), _vp(up), _vp(act), gate.numel(), s), "swiglu")
            return self._rows_linears(layer, (name,), act)[0]
        self._check(lib.sageb200_glue_swiglu_permuted(_vp(gate), _vp(up), _vp(permutation), _vp(act), gate.numel() // k, k,
                                                      self.sm_count, s), "swiglu_permuted")
        return self._pregathered(layer[name], act)

    def _rows_linears(self, layer, names, x):
        if self.dense:
            return [torch.nn.functional.linear(x, layer[name].weight) for name in names]
        if x.dim() == 2 and 16 < x.shape[0] <= 32 and 2 * len(names) <= _lib.MAX_GROUPED:
            linears = [layer[name] for name in names]
            return self._grouped_row_blocks(linears, x, [linear.packed["permutation"] for linear in linears])
        return [self._packed_rows(layer[name], x, layer[name].packed["permutation"]) for name in names]

    def _prefill_batched(self, prompt: torch.Tensor):
        if self.tp_world > 1 or self.ep_world > 1 or self.config.experts:
            raise ValueError("batched prefill runs on one GPU with a dense-MLP config")
        c, lib, b = self.config, self.lib, self.batch
        length = prompt.shape[1]
        rows = b * length  # row = sequence * length + token
        half = dict(dtype=torch.float16, device=self.device)
        with torch.cuda.device(self.device):
            s = self._stream()
            tokens = prompt.reshape(-1).to(torch.int64).contiguous()
            h = torch.empty(rows, c.hidden, **half)
            attn = torch.empty(rows, self.heads * c.head_dim, **half)
            self._check(lib.sageb200_glue_embed(_vp(self.embed), _vp(tokens), _vp(h), rows, c.hidden, c.vocab, s), "embed")
            delta = None
            for layer in self.layers:
                q, k, v = self._norm_rows_linears(layer, ("q", "k", "v"), h, delta, layer["input_norm"], rows)
                self._check(lib.sageb200_glue_prefill_qk_norm_rope_cache(
                    _vp(q), _vp(k), _vp(v), _vp(layer["q_norm"]), _vp(layer["k_norm"]), _vp(self.cos), _vp(self.sin),
                    _vp(self.positions), _vp(layer["k_cache"]), _vp(layer["v_cache"]), b, length, self.heads,
                    self.kv_heads, c.head_dim, self.max_seq, c.eps, s), "prefill_qk_norm_rope_cache")
                self._check(lib.sageb200_glue_prefill_attention(
                    _vp(q), _vp(layer["k_cache"]), _vp(layer["v_cache"]), _vp(self.positions), _vp(attn), b, length,
                    self.heads, self.kv_heads, c.head_dim, self.max_seq, s), "prefill_attention")
                (o,) = self._rows_linears(layer, ("o",), attn)
                gate, up = self._norm_rows_linears(layer, ("gate", "up"), h, o, layer["post_norm"], rows)
                delta = self._swiglu_rows_linear(layer, "down", gate, up)
            # the step tail on each sequence's last prompt token
            last = torch.arange(b, device=self.device) * length + (length - 1)
            h_last, delta_last = h[last].contiguous(), delta[last].contiguous()
            self.positions.add_(length - 1)
            self._tail(h_last, delta_last)

    def generate(self, prompt: torch.Tensor, new_tokens: int) -> torch.Tensor:
        """Greedy generation; returns [batch, new_tokens] token ids (device tensor)."""
        if new_tokens > self.max_new:
            raise ValueError("new_tokens exceeds max_new")
        if prompt.shape[1] + new_tokens - 1 > self.max_seq:
            raise ValueError(f"prompt ({prompt.shape[1]}) + new tokens ({new_tokens}) exceed the cache of "
                             f"{self.max_seq} positions")
        self.prefill(prompt)  # logs token 0
        for _ in range(new_tokens - 1):
            self.graph.replay()
        return self.log[:, :new_tokens].clone()

    def bytes_per_token(self, context: int) -> int:
        """Algorithmic HBM bytes of one decode iteration at batch 1: packed linears, FP16
        lm_head, KV cache read for `context` positions."""
        c = self.config
        kv = 2 * c.layers * self.kv_heads * c.head_dim * 2 * context
        return self.packed_bytes + (c.vocab // self.tp_world) * c.hidden * 2 + kv
