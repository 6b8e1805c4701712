"""Peer-memory plumbing for the window-parallel halo exchange.

Each WP rank owns one symmetric staging buffer (allocated through ``torch.distributed._symmetric_memory``, i.e. CUDA
VMM + handle exchange) that its peers can read with plain loads over NVLink. A re-partition between the plain and the
shifted window layout then is: publish this rank's rows in the staging buffer -> rank barrier -> every rank's gather
kernel pulls the rows it needs straight from the owners' buffers (local HBM or peer HBM) -> rank barrier. The pull is
done by the same row-gather kernels that do the local re-partition, so no send/recv buffers, packing kernels or
rolls exist (reference: blocking send/recv of three strips + ``torch.roll`` per shift,
src/aeris_wp_inference/model.py:72-114).
"""
from __future__ import annotations

import torch
import torch.distributed as dist


class HaloExchange:
    def __init__(self, group, device):
        self.group = group
        self.device = torch.device(device)
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self._buf = None
        self._hdl = None
        self._flag = torch.zeros(1, device=self.device)

    def _ensure(self, numel: int, dtype: torch.dtype):
        if self._buf is not None and self._buf.numel() >= numel and self._buf.dtype == dtype:
            return
        import torch.distributed._symmetric_memory as symm_mem
        self._buf = symm_mem.empty(numel, dtype=dtype, device=self.device)
        self._hdl = symm_mem.rendezvous(self._buf, self.group)
        self._peer_ptrs = [int(p) for p in self._hdl.buffer_ptrs]

    def _barrier(self):
        # stream-ordered rank barrier (tiny NCCL all-reduce on the current stream)
        dist.all_reduce(self._flag, group=self.group)

    def peer_fn(self, src: torch.Tensor, direction: str) -> list[int]:
        """Publishes ``src`` (this rank's rows) and returns every rank's staging-buffer address. The caller launches
        its gather right after; :meth:`release` must follow it before the next publish."""
        self._ensure(src.numel(), src.dtype)
        self._barrier()                      # peers finished reading the previous contents
        self._buf[:src.numel()].view_as(src).copy_(src)
        self._barrier()                      # every rank's rows are visible
        return self._peer_ptrs
