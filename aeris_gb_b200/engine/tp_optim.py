"""Optimizer of a model whose MLP weights are tensor-parallel shards.

Two kinds of parameters live on every rank of the weight group (the WP x SP x DP ranks that hold one model replica
between them):
  * replicated ones (attention, norms, modulation, input and output stage): their gradients are partial sums over the
    rank's tokens and are reduced over the whole weight group, by the sharded peer-memory optimizer or by NCCL;
  * tensor-parallel shards (``w1`` / ``w2`` of every block): the fused MLP kernels already accumulate the gradient
    over the token rows of every rank of the tensor-parallel group, so it is reduced only over the ranks that hold the
    SAME shard (``ortho_group``; nothing to do when the tensor-parallel group is the whole weight group).
Both share one clipping norm: sum of squares of the replicated gradients plus the sum over the tensor-parallel ranks
of their shards' squares. State dicts carry FULL tensors for the shards (gathered over the tensor-parallel group), so
checkpoints do not depend on the tensor-parallel degree; loading cuts them again.

The reference has no tensor parallelism; the replicated half is its optimizer mode (a) / (b) of
src/aeris/parallelism/parallel_engine.py:702-792.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn

from ..parallel.tensor import fit_to_shard, full_state_dict, tp_kind
from .optim import FlatOptimizer, OptimConfig


class TPOptimizer:
    def __init__(self, model: nn.Module, cfg: OptimConfig, device, weight_group, tp_group, ortho_group=None,
                 fused: bool = False, use_multicast: bool = False):
        self.cfg, self.device = cfg, torch.device(device)
        self.weight_group, self.tp_group, self.ortho_group = weight_group, tp_group, ortho_group
        self.tp, self.tp_rank = dist.get_world_size(tp_group), dist.get_rank(tp_group)
        named = [(n, p) for n, p in model.named_parameters() if p.requires_grad]
        tp_named = [(n, p) for n, p in named if tp_kind(n, p) is not None]
        rep_named = [(n, p) for n, p in named if tp_kind(n, p) is None]
        assert tp_named, "the model holds no tensor-parallel shards (AerisConfig.tp == 1?)"
        self.fused = fused
        if fused:
            from .fused_dp import FusedShardedOptimizer
            self.rep = FusedShardedOptimizer(model, cfg, weight_group, device, use_multicast, params=rep_named)
        else:
            self.rep = FlatOptimizer(model, cfg, params=rep_named)
        self.tpo = FlatOptimizer(model, cfg, params=tp_named)
        self.host_copies = True
        self.last_lr = 0.0

    # ---- the optimizer interface the trainer and the checkpoint code use ------------------------------------------------
    @property
    def step_count(self) -> int:
        return self.rep.step_count

    @property
    def cur_nimg(self) -> int:
        return self.rep.cur_nimg

    @property
    def uses_multicast(self) -> bool:
        return bool(getattr(self.rep, "uses_multicast", False))

    def grad_buffers(self):
        return list(self.rep.grad_buffers()) + list(self.tpo.grad_buffers())

    def zero_grad(self):
        self.rep.zero_grad()
        self.tpo.zero_grad()

    def reduce_and_step(self, batch_img: int, grad_scale: float) -> torch.Tensor | None:
        c = self.cfg
        if self.ortho_group is not None and dist.get_world_size(self.ortho_group) > 1:
            for buf in self.tpo.grad_buffers():
                dist.all_reduce(buf, group=self.ortho_group)
        nsq_tp = None
        if c.grad_clip:
            nsq_tp = self.tpo.grad_norm_sq(grad_scale).clone()
            dist.all_reduce(nsq_tp, group=self.tp_group)
        if self.fused:
            total = self.rep.reduce_and_step(batch_img, grad_scale, extra_sumsq=nsq_tp)
            if not c.grad_clip:
                total = None
        else:
            for buf in self.rep.grad_buffers():
                dist.all_reduce(buf, group=self.weight_group)
            total = (self.rep.grad_norm_sq(grad_scale) + nsq_tp) if c.grad_clip else None
            self.rep.step(batch_img=batch_img, grad_scale=grad_scale, norm_sq=total)
        self.tpo.step(batch_img=batch_img, grad_scale=grad_scale, norm_sq=total)
        self.last_lr = self.tpo.last_lr
        return total

    # ---- the same update in the three phases the pipeline engine drives (NCCL / gloo collectives only) -----------------
    def reduce(self, group=None):
        assert not self.fused, "the peer-memory optimizer reduces inside reduce_and_step"
        if self.ortho_group is not None and dist.get_world_size(self.ortho_group) > 1:
            for buf in self.tpo.grad_buffers():
                dist.all_reduce(buf, group=self.ortho_group)
        if self.weight_group is not None:
            for buf in self.rep.grad_buffers():
                dist.all_reduce(buf, group=self.weight_group)

    def grad_norm_sq(self, grad_scale: float) -> torch.Tensor:
        """Squared norm of this stage's reduced, scaled gradient: replicated parameters once, shards summed over the
        tensor-parallel group."""
        nsq_tp = self.tpo.grad_norm_sq(grad_scale).clone()
        dist.all_reduce(nsq_tp, group=self.tp_group)
        return self.rep.grad_norm_sq(grad_scale) + nsq_tp

    def step(self, batch_img: int, grad_scale: float, norm_sq: torch.Tensor | None = None):
        self.rep.step(batch_img=batch_img, grad_scale=grad_scale, norm_sq=norm_sq)
        self.tpo.step(batch_img=batch_img, grad_scale=grad_scale, norm_sq=norm_sq)
        self.last_lr = self.tpo.last_lr

    # ---- state: replicated entries as the inner optimizer gives them, shards gathered to full tensors ----------------
    def _full(self, named: dict) -> dict:
        return full_state_dict(named, self.tp_group)

    def _merge(self, which: str) -> dict:
        if hasattr(self.rep, "host_copies"):
            self.rep.host_copies = self.host_copies
        out = dict(getattr(self.rep, which)())
        out.update(self._full(getattr(self.tpo, which)()))
        return out

    def master_state_dict(self) -> dict:
        return self._merge("master_state_dict")

    def ema_state_dict(self) -> dict:
        return self._merge("ema_state_dict")

    def state_dict(self) -> dict:
        if hasattr(self.rep, "host_copies"):
            self.rep.host_copies = self.host_copies
        a, b = self.rep.state_dict(), self.tpo.state_dict()
        return {"step": a["step"], "cur_nimg": a["cur_nimg"],
                "exp_avg": {**a["exp_avg"], **self._full(b["exp_avg"])},
                "exp_avg_sq": {**a["exp_avg_sq"], **self._full(b["exp_avg_sq"])}}

    def load_state_dict(self, sd: dict, master: dict | None = None, ema: dict | None = None):
        like = self.tpo.master_state_dict()

        def cut(named):
            if named is None:
                return None
            return {k: fit_to_shard(k, t, like[k], self.tp, self.tp_rank) for k, t in named.items() if k in like}

        self.rep.load_state_dict(sd, master=master, ema=ema)
        self.tpo.load_state_dict({"step": sd["step"], "cur_nimg": sd["cur_nimg"], "exp_avg": cut(sd.get("exp_avg")) or {},
                                  "exp_avg_sq": cut(sd.get("exp_avg_sq")) or {}}, master=cut(master), ema=cut(ema))
