"""ZeRO-1-style distributed optimizer over the weight group.

Reference (src/aeris/parallelism/parallel_engine.py:126-135, 743-792, 834-860, 1321-1397): one flat bf16 buffer that
is both gradient accumulator and all-gather target, the optimizer built on this rank's shard, reduce-scatter (or
all-reduce + slice) of gradients, all-gather of updated parameters, no fp32 master, no EMA, no checkpoint. Here the
shard keeps fp32 master weights, Adam moments and (optionally) the EMA, gradients stay fp32 until reduced, the
sharded state can be checkpointed, and the update itself is the same fused AdamW kernel as in the local optimizer.
"""
from __future__ import annotations

import math
import os

import torch
import torch.distributed as dist

from .optim import FlatOptimizer, OptimConfig, ema_beta_at, lr_at


class DistOptimizer(FlatOptimizer):
    def __init__(self, model, cfg: OptimConfig, group, rs_grads: bool = True):
        super().__init__(model, cfg)
        self.group = group
        self.rs_grads = rs_grads
        self.world = dist.get_world_size(group) if group is not None else 1
        self.grank = dist.get_rank(group) if group is not None else 0
        # shard every segment: padded to a multiple of the group size; this rank keeps [lo, hi)
        for s in self.segments:
            per = math.ceil(s.numel / self.world)
            per = (per + 15) // 16 * 16
            s.shard = per
            s.lo = self.grank * per
            pad = per * self.world - s.numel
            if pad:
                def grow(t):
                    return torch.cat([t, torch.zeros(pad, dtype=t.dtype, device=t.device)])
                # the parameters keep pointing into the (now longer) flat buffers: re-create the views
                old_grad, old_master, old_flat = s.grad, s.master, s.model_flat
                s.grad, s.master = grow(s.grad), grow(s.master)
                if s.model_flat is not None:
                    s.model_flat = grow(s.model_flat)
                off = 0
                for p in s.params:
                    n = p.numel()
                    target = s.model_flat if s.low_precision else s.master
                    p.data = target[off:off + n].view(p.shape)
                    p.main_grad = s.grad[off:off + n].view(p.shape)
                    off += (n + 15) // 16 * 16
                del old_grad, old_master, old_flat
            sl = slice(s.lo, s.lo + per)
            s.master_shard = s.master[sl].clone()
            s.m, s.v = torch.zeros_like(s.master_shard), torch.zeros_like(s.master_shard)
            s.ema = s.master_shard.clone() if cfg.use_ema else None
            s.grad_shard = torch.zeros_like(s.master_shard)
            s.out_shard = torch.zeros(per, dtype=s.model_flat.dtype, device=s.master.device) if s.low_precision else None

    def reduce(self, group=None):
        """Reduce-scatter (or all-reduce + slice, ``rs_grads=False``) of the accumulated gradients into the shard."""
        for s in self.segments:
            if self.world == 1:
                s.grad_shard.copy_(s.grad[s.lo:s.lo + s.shard])
            elif self.rs_grads and dist.get_backend(self.group) == "nccl":
                dist.reduce_scatter_tensor(s.grad_shard, s.grad, group=self.group)
            else:
                dist.all_reduce(s.grad, group=self.group)
                s.grad_shard.copy_(s.grad[s.lo:s.lo + s.shard])
            s.grad.zero_()

    def grad_norm_sq(self, grad_scale: float) -> torch.Tensor:
        dev = self.segments[0].grad.device
        nsq = torch.zeros(1, dtype=torch.float64, device=dev)
        for s in self.segments:
            nsq += s.grad_shard.double().pow(2).sum()
        if self.world > 1:
            dist.all_reduce(nsq, group=self.group)
        nsq *= grad_scale * grad_scale
        return nsq

    def step(self, batch_img: int, grad_scale: float, norm_sq=None):
        c = self.cfg
        self.step_count += 1
        lr = lr_at(self.cur_nimg, c.lr, c)
        beta = ema_beta_at(self.cur_nimg, batch_img, c) if c.use_ema else None
        max_norm = c.grad_clip_max_norm if (c.grad_clip and norm_sq is not None) else 0.0
        for s in self.segments:
            wd = c.weight_decay if s.decay else 0.0
            if s.master_shard.is_cuda:
                from ..ops import elementwise as E
                E.adamw(s.master_shard, s.grad_shard, s.m, s.v, s.out_shard, s.ema if beta is not None else None,
                        norm_sq, lr=lr, betas=c.betas, eps=c.eps, weight_decay=wd, step=self.step_count,
                        grad_scale=grad_scale, max_norm=max_norm, ema_beta=beta if beta is not None else -1.0)
            else:
                view = type("S", (), {})()
                view.grad, view.m, view.v, view.master, view.ema = s.grad_shard, s.m, s.v, s.master_shard, s.ema
                view.model_flat = s.out_shard
                self._step_cpu(view, lr, wd, grad_scale, max_norm, norm_sq, beta)
            # all-gather the updated parameters into every rank's full buffer
            target = s.model_flat if s.low_precision else s.master
            src = s.out_shard if s.low_precision else s.master_shard
            if self.world > 1:
                dist.all_gather_into_tensor(target, src, group=self.group) if dist.get_backend(self.group) == "nccl" \
                    else self._gather_gloo(target, src)
            else:
                target[s.lo:s.lo + s.shard].copy_(src)
        self.cur_nimg += batch_img
        self.last_lr = lr

    def _gather_gloo(self, target, src):
        parts = [torch.empty_like(src) for _ in range(self.world)]
        dist.all_gather(parts, src, group=self.group)
        target.copy_(torch.cat(parts))

    # ---- state for checkpoints: gathered over the group (collective), in the layout of FlatOptimizer ----------------
    host_copies = True      # False on ranks that only take part in the gathers of a checkpoint another rank writes

    def _gather_full(self, s, which: str) -> torch.Tensor | None:
        shard = {"m": s.m, "v": s.v, "master": s.master_shard, "ema": s.ema}[which]
        if shard is None:
            return None
        if self.world == 1:
            return shard
        if dist.get_backend(self.group) == "nccl":
            full = torch.empty(s.shard * self.world, dtype=shard.dtype, device=shard.device)
            dist.all_gather_into_tensor(full, shard.contiguous(), group=self.group)
        else:
            parts = [torch.empty_like(shard) for _ in range(self.world)]
            dist.all_gather(parts, shard.contiguous(), group=self.group)
            full = torch.cat(parts)
        return full.cpu() if self.host_copies else None

    def _named_views(self, which: str) -> dict[str, torch.Tensor]:
        out = {}
        for s in self.segments:
            full = self._gather_full(s, which)
            if full is None:
                continue
            off = 0
            for n, p in zip(s.names, s.params):
                out[n] = full[off:off + p.numel()].view(p.shape)
                off += (p.numel() + 15) // 16 * 16
        return out

    def load_state_dict(self, sd: dict, master: dict | None = None, ema: dict | None = None):
        """Every rank reads the full named arrays and keeps its shard; the working copy of the weights is rebuilt from
        the masters on every rank."""
        self.step_count, self.cur_nimg = int(sd["step"]), int(sd["cur_nimg"])
        sources = {"m": sd.get("exp_avg"), "v": sd.get("exp_avg_sq"), "master": master, "ema": ema}
        for s in self.segments:
            for which, named in sources.items():
                dst = {"m": s.m, "v": s.v, "master": s.master_shard, "ema": s.ema}[which]
                if named is None or dst is None:
                    continue
                off = 0
                for n, p in zip(s.names, s.params):
                    cnt = p.numel()
                    if n in named:
                        src = named[n].reshape(-1).to(dst.device, torch.float32)
                        a, b = max(off, s.lo), min(off + cnt, s.lo + s.shard)      # overlap with this rank's shard
                        if a < b:
                            dst[a - s.lo:b - s.lo].copy_(src[a - off:b - off])
                        if which == "master":
                            s.master[off:off + cnt].copy_(src)
                            if s.model_flat is not None:
                                s.model_flat[off:off + cnt].copy_(src.to(s.model_flat.dtype))
                    off += (cnt + 15) // 16 * 16
