"""All-reduce of row-parallel partial outputs over the peers' memory (one node, one process
per GPU): the host side of include/sage_b200_peer.h.

`PeerExchange` allocates this rank's exchange, swaps the IPC handles over the process group and
maps the peers' exchanges; `all_reduce(tensor)` is then one kernel per rank (push over NVLink,
epoch flags, sum in rank order) that can be captured in a CUDA graph.  The reference has no
multi-GPU packed inference; the row/column split follows weight_vq/blockwise/artifacts.py:10-18.
"""

from __future__ import annotations

import ctypes

import torch

from . import _lib


class PeerExchange:
    """Exchange buffers of one process group on one node.  Every rank must construct it with the
    same `capacity` (FP16 elements of the largest tensor to reduce) and make the same sequence
    of `all_reduce` calls."""

    def __init__(self, group, device, capacity: int):
        import torch.distributed as dist

        self.lib = _lib.load()
        self.group = group
        self.device = torch.device(device)
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if not 2 <= self.world <= _lib.PEER_MAX_WORLD:
            raise ValueError(f"a peer exchange serves 2..{_lib.PEER_MAX_WORLD} ranks")
        self.capacity = (int(capacity) + 7) // 8 * 8
        self.own = ctypes.c_void_p()
        self.exchanges = (ctypes.c_void_p * _lib.PEER_MAX_WORLD)()
        self.opened = []
        handle = (ctypes.c_ubyte * _lib.PEER_HANDLE_BYTES)()
        with torch.cuda.device(self.device):
            # Every rank runs every collective below whatever happens to it, and the ranks agree on
            # the outcome at the end, so that a rank that cannot allocate or map (IPC not permitted
            # in this container, peer access unavailable) makes ALL ranks raise together instead
            # of leaving the others waiting on flags nobody will publish.
            failure = ""
            status = self.lib.sageb200_peer_create(self.world, self.capacity, ctypes.byref(self.own), handle)
            if status != _lib.OK:
                failure = f"sageb200_peer_create failed with status {status}"
                self.own = ctypes.c_void_p()
            mine = torch.tensor(list(handle), dtype=torch.uint8, device=self.device)
            everyone = torch.empty(self.world * _lib.PEER_HANDLE_BYTES, dtype=torch.uint8, device=self.device)
            dist.all_gather_into_tensor(everyone, mine, group=group)
            handles = everyone.cpu().view(self.world, _lib.PEER_HANDLE_BYTES)
            created = torch.tensor([0 if failure else 1], dtype=torch.int32, device=self.device)
            dist.all_reduce(created, op=dist.ReduceOp.MIN, group=group)
            if int(created) == 1:
                for r in range(self.world):
                    if r == self.rank:
                        self.exchanges[r] = self.own.value
                        continue
                    raw = (ctypes.c_ubyte * _lib.PEER_HANDLE_BYTES)(*handles[r].tolist())
                    mapped = ctypes.c_void_p()
                    status = self.lib.sageb200_peer_open(raw, ctypes.byref(mapped))
                    if status != _lib.OK:
                        failure = failure or f"sageb200_peer_open of rank {r}'s exchange failed with status {status}"
                        continue
                    self.exchanges[r] = mapped.value
                    self.opened.append(mapped.value)
            elif not failure:
                failure = "another rank could not allocate its exchange"
            # nobody launches before every rank has mapped every exchange
            agreed = torch.tensor([0 if failure else 1], dtype=torch.int32, device=self.device)
            dist.all_reduce(agreed, op=dist.ReduceOp.MIN, group=group)
            if int(agreed) != 1:
                for mapped in self.opened:
                    self.lib.sageb200_peer_close(ctypes.c_void_p(mapped))
                dist.barrier(group=group)
                if self.own.value:
                    self.lib.sageb200_peer_destroy(self.own)
                self.own = None
                raise RuntimeError("sage_b200: peer exchange unavailable: " + (failure or "another rank failed to map a peer"))
            dist.barrier(group=group)
        self.calls = 0

    def all_reduce(self, tensor: torch.Tensor) -> torch.Tensor:
        """In place: `tensor` (FP16, contiguous, numel a multiple of 8 and at most `capacity`)
        becomes the sum over the ranks, identical on every rank."""
        if tensor.dtype != torch.float16 or not tensor.is_contiguous() or tensor.device != self.device:
            raise ValueError("the peer all-reduce takes a contiguous FP16 tensor on the exchange's device")
        stream = torch.cuda.current_stream(self.device).cuda_stream
        _lib.check(self.lib.sageb200_peer_all_reduce(self.exchanges, self.world, self.rank, self.capacity,
                                                     tensor.data_ptr(), tensor.numel(), stream))
        self.calls += 1
        return tensor

    def fits(self, tensor: torch.Tensor) -> bool:
        return tensor.dtype == torch.float16 and tensor.numel() % 8 == 0 and 0 < tensor.numel() <= self.capacity

    def close(self):
        """Collective: every rank's kernels on the exchange must have finished (synchronises)."""
        import torch.distributed as dist

        if self.own is None:
            return
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        with torch.cuda.device(self.device):
            for mapped in self.opened:
                self.lib.sageb200_peer_close(ctypes.c_void_p(mapped))
            dist.barrier(group=self.group)
            self.lib.sageb200_peer_destroy(self.own)
        self.own = None
