"""Point-to-point links of one pipeline rank (NCCL on GPUs, gloo on CPU).

The reference moves activations and gradients between stages with blocking ``send`` / ``recv`` on pairwise groups
(src/aeris/parallelism/parallel_engine.py:1026,1034,425-451) or, in its overlapped mode, with MPI ``Isend`` / ``Irecv``
through host memory (:1022-1032). Here every link has one communicator per direction (``down``: activations,
``up``: gradients; :meth:`ProcessGrid.build_groups`), every transfer is one grouped ``batch_isend_irecv`` (x and dt
travel in one NCCL launch), and nothing waits on the host: a receive is posted when the schedule says so (one step
early in the overlapped schedule), the consumer's stream waits for it, sends are never waited for before the end of the
step. NCCL runs each communicator on a stream of its own, which it orders after the work queued on the compute stream
at issue time: a send waits for the kernel that produced its tensor, a receive posted before this step's kernels runs
beside them.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


class PipeLinks:
    def __init__(self, groups: dict, prev_rank: int | None, next_rank: int | None, device,
                 result_peer: int | None = None):
        self.groups, self.device = groups, device
        self.peer = {"down_next": next_rank, "up_next": next_rank, "down_prev": prev_rank, "up_prev": prev_rank,
                     "result": result_peer}
        self._sends: list = []       # (work handles, tensors kept alive until the transfer is done)
        self.n_ops = {k: 0 for k in self.peer}

    def warm(self) -> None:
        """One tiny transfer per channel in a fixed order (down the pipeline, then up), so that communicators created
        on first use come up pair by pair before the schedule runs."""
        one = torch.zeros(1, device=self.device)
        for ch, kind in (("down_prev", "recv"), ("down_next", "send"), ("up_next", "recv"), ("up_prev", "send")):
            if self.peer[ch] is not None and self.groups.get(ch) is not None:
                for w in self._issue(ch, kind, [one]):
                    w.wait()
        if self.device.type == "cuda":
            torch.cuda.synchronize()

    def _issue(self, channel: str, kind: str, tensors: list[torch.Tensor]):
        fn = dist.isend if kind == "send" else dist.irecv
        ops = [dist.P2POp(fn, t, self.peer[channel], group=self.groups[channel]) for t in tensors]
        self.n_ops[channel] += len(ops)
        return dist.batch_isend_irecv(ops)

    def send(self, channel: str, tensors: list[torch.Tensor]) -> None:
        tensors = [t.detach().contiguous() for t in tensors]
        self._sends = [(ws, ts) for ws, ts in self._sends if not all(w.is_completed() for w in ws)]
        self._sends.append((self._issue(channel, "send", tensors), tensors))

    def post_recv(self, channel: str, tensors: list[torch.Tensor]):
        """Returns the handles; :meth:`wait` makes the current stream (gloo: the host) wait for the data."""
        return self._issue(channel, "recv", tensors)

    @staticmethod
    def wait(works) -> None:
        for w in works:
            w.wait()

    def wait_sends(self) -> None:
        for ws, _ in self._sends:
            self.wait(ws)
        self._sends = []
