"""Peer-memory plumbing for the window-parallel halo exchange.

Each WP rank owns one symmetric staging buffer (allocated through ``torch.distributed._symmetric_memory``, i.e. CUDA
VMM + handle exchange) that its peers can read with plain loads over NVLink. A re-partition between the plain and the
shifted window layout then is: publish this rank's rows in the staging buffer -> rank barrier -> every rank's gather
kernel pulls the rows it needs straight from the owners' buffers (local HBM or peer HBM) -> rank barrier. The pull is
done by the same row-gather kernels that do the local re-partition, so no send/recv buffers, packing kernels or
rolls exist (reference: blocking send/recv of three strips + ``torch.roll`` per shift,
src/aeris_wp_inference/model.py:72-114).

Producers that know their output will be re-partitioned next (the last block of a Swin layer, the gradient gather of
the layer after it) write it straight into one of two alternating symmetric buffers (:meth:`output_buffer`); publishing
such a tensor needs no copy and a single barrier. Two buffers suffice: a rank can only overwrite buffer b two
re-partitions later, and it passes the barrier of the re-partition in between only after every peer has finished
reading buffer b.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


class HaloExchange:
    def __init__(self, group, device, pool_gradients: bool = True):
        # pool_gradients=False: gathered gradients get ordinary buffers (for engines that hand them to asynchronous
        # sends, which must not see the buffer recycled two re-partitions later)
        self.pool_gradients = pool_gradients
        self.group = group
        self.device = torch.device(device)
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self._buf = None
        self._hdl = None
        self._flag = torch.zeros(1, device=self.device)
        import os
        self._nccl_barrier = os.environ.get("AERIS_HALO_NCCL_BARRIER") == "1"
        self._rank_barrier = None
        self._pool: list[torch.Tensor] = []       # two alternating symmetric output buffers
        self._pool_ptrs: list[list[int]] = []
        self._pool_hdl: list = []
        self._turn = 0
        self.timers = None            # utils.timers.DeviceTimers: when enabled, the barriers are timed as "halo_barrier"

    def _ensure(self, numel: int, dtype: torch.dtype):
        if self._buf is not None and self._buf.numel() >= numel and self._buf.dtype == dtype:
            return
        import torch.distributed._symmetric_memory as symm_mem
        self._buf = symm_mem.empty(numel, dtype=dtype, device=self.device)
        self._hdl = symm_mem.rendezvous(self._buf, self.group)
        self._peer_ptrs = [int(p) for p in self._hdl.buffer_ptrs]

    def _barrier(self):
        """Stream-ordered rank barrier: epoch flags in peer memory (one small kernel, release stores to every peer and
        a bounded acquire spin on the own flags), or with AERIS_HALO_NCCL_BARRIER=1 a one-element NCCL all-reduce."""
        if self.timers is not None and self.timers.enabled:
            with self.timers.region("halo_barrier"):      # device time of the flag kernel = arrival skew of the ranks
                self._barrier_now()
        else:
            self._barrier_now()

    def _barrier_now(self):
        if self._nccl_barrier:
            dist.all_reduce(self._flag, group=self.group)
            return
        if self._rank_barrier is None:
            from ..engine.fused_dp import RankBarrier
            self._rank_barrier = RankBarrier(self.group, self.device)
        self._rank_barrier()

    def output_buffer(self, rows: int, cols: int, dtype: torch.dtype) -> torch.Tensor:
        """``[rows, cols]`` tensor inside the symmetric buffer whose turn it is (collective on first use and whenever a
        larger size is asked for: every rank asks for the same sizes in the same order)."""
        numel = rows * cols
        if not self._pool or self._pool[0].numel() < numel or self._pool[0].dtype != dtype:
            import torch.distributed._symmetric_memory as symm_mem
            self._pool, self._pool_ptrs, self._pool_hdl = [], [], []
            for _ in range(2):
                t = symm_mem.empty(numel, dtype=dtype, device=self.device)
                hdl = symm_mem.rendezvous(t, self.group)
                self._pool.append(t)
                self._pool_hdl.append(hdl)
                self._pool_ptrs.append([int(p) for p in hdl.buffer_ptrs])
        self._turn ^= 1
        return self._pool[self._turn][:numel].view(rows, cols)

    def gradient_buffer(self, rows: int, cols: int, dtype: torch.dtype) -> torch.Tensor:
        """Where a gathered gradient goes: a pooled peer-readable buffer, or an ordinary one (see ``pool_gradients``)."""
        if self.pool_gradients:
            return self.output_buffer(rows, cols, dtype)
        return torch.empty((rows, cols), dtype=dtype, device=self.device)

    def _pool_slot(self, src: torch.Tensor):
        p = src.data_ptr()
        for b, t in enumerate(self._pool):
            lo = t.data_ptr()
            if lo <= p and p + src.numel() * src.element_size() <= lo + t.numel() * t.element_size():
                return b, p - lo
        return None

    def peer_fn(self, src: torch.Tensor, direction: str) -> list[int]:
        """Publishes ``src`` (this rank's rows) and returns, for every rank, the address of its copy of those rows. The
        caller launches its gather right after. A ``src`` that already lives in one of the :meth:`output_buffer`s is
        published in place."""
        slot = self._pool_slot(src) if src.is_contiguous() else None
        if slot is not None:
            b, off = slot
            self._barrier()                  # every rank has finished writing its rows
            return [p + off for p in self._pool_ptrs[b]]
        self._ensure(src.numel(), src.dtype)
        self._barrier()                      # peers finished reading the previous contents
        self._buf[:src.numel()].view_as(src).copy_(src)
        self._barrier()                      # every rank's rows are visible
        return self._peer_ptrs
