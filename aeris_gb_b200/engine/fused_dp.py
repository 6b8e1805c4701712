"""Sharded optimizer whose collectives are this library's own peer-memory kernels (``csrc/comm.cu``).

For the ranks that hold replicas of the same weights on one NVSwitch node (the weight group: WP x SP x DP):
  * the flat fp32 gradient buffer and the flat bf16 parameter buffer live in symmetric memory;
  * each rank owns 1/world of the fp32 master weights, Adam moments and EMA (ZeRO-1 memory saving);
  * step = [rank barrier] -> fused reduce-scatter + scale + sum-of-squares kernel (pulls the shard from every peer, or
    one ``multimem.ld_reduce`` through the switch) -> one scalar all-reduce for the clip norm -> fused AdamW kernel that
    writes the updated bf16 weights into every peer's parameter buffer (the all-gather is the store) -> [rank barrier].
Reference counterpart: reduce_scatter / all_reduce, scaling, clipping, optimizer.step and all_gather as separate calls
(src/aeris/parallelism/parallel_engine.py:743-792, 832-859). fp32 parameters (input and output stage, a few hundred
thousand values) are not sharded; they take an ordinary NCCL all-reduce and the local fused AdamW kernel.
"""
from __future__ import annotations

import ctypes
import math

import torch
import torch.distributed as dist
import torch.nn as nn

from ..ops import elementwise as E
from ..ops import lib as L
from .optim import OptimConfig, ema_beta_at, lr_at, no_decay_names


def _ptr_array(ptrs):
    return (ctypes.c_void_p * len(ptrs))(*ptrs)


class RankBarrier:
    """Stream-ordered barrier between the ranks of a node through flag words in symmetric memory (bounded wait)."""

    def __init__(self, group, device, timeout_s: float = 20.0):
        import torch.distributed._symmetric_memory as symm_mem
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.flags = symm_mem.empty(32, dtype=torch.int32, device=device)
        self.flags.zero_()
        self.hdl = symm_mem.rendezvous(self.flags, group)
        self.ptrs = _ptr_array([int(p) for p in self.hdl.buffer_ptrs])
        self.epoch, self.timeout_s = 0, timeout_s
        dist.barrier(group)      # every rank's flags are zeroed before the first epoch is written

    def __call__(self):
        self.epoch += 1
        rc = L.lib().aeris_signal_barrier(self.ptrs, self.rank, self.world, ctypes.c_uint(self.epoch),
                                          L.ptr(L.status_word()), ctypes.c_double(self.timeout_s), L.stream_ptr())
        L.check(rc, "aeris_signal_barrier")


class _Seg:
    pass


class FusedShardedOptimizer:
    def __init__(self, model: nn.Module, cfg: OptimConfig, group, device, use_multicast: bool = True, params=None):
        """``params``: the (name, parameter) pairs to manage; default: every trainable parameter of ``model``."""
        import torch.distributed._symmetric_memory as symm_mem
        self.cfg, self.group, self.device = cfg, group, torch.device(device)
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.step_count, self.cur_nimg = 0, 0
        nd = no_decay_names(model, cfg.decay_policy)
        segs: dict[tuple[bool, bool], _Seg] = {}
        for n, p in (params if params is not None else model.named_parameters()):
            if not p.requires_grad:
                continue
            key = (p.dtype != torch.float32, n not in nd)
            if key not in segs:
                s = _Seg()
                s.low_precision, s.decay, s.params, s.names = key[0], key[1], [], []
                segs[key] = s
            segs[key].params.append(p)
            segs[key].names.append(n)
        self.segments = list(segs.values())
        self.barrier = RankBarrier(group, self.device)
        for s in self.segments:
            offs, total = [], 0
            for p in s.params:
                offs.append(total)
                total += (p.numel() + 15) // 16 * 16
            s.offs, s.numel = offs, total
            if s.low_precision:
                per = (math.ceil(total / self.world) + 15) // 16 * 16
                s.per, s.lo, s.padded = per, self.rank * per, per * self.world
                s.grad = symm_mem.empty(s.padded, dtype=torch.float32, device=self.device)
                s.grad.zero_()
                s.model_flat = symm_mem.empty(s.padded, dtype=s.params[0].dtype, device=self.device)
                s.model_flat.zero_()
                s.grad_hdl = symm_mem.rendezvous(s.grad, group)
                s.param_hdl = symm_mem.rendezvous(s.model_flat, group)
                s.grad_ptrs = _ptr_array([int(x) for x in s.grad_hdl.buffer_ptrs])
                s.param_ptrs = _ptr_array([int(x) for x in s.param_hdl.buffer_ptrs])
                s.mc_grad = int(getattr(s.grad_hdl, "multicast_ptr", 0) or 0) if use_multicast else 0
                s.mc_param = int(getattr(s.param_hdl, "multicast_ptr", 0) or 0) if use_multicast else 0
                full_master = torch.zeros(s.padded, dtype=torch.float32, device=self.device)
                for p, off in zip(s.params, offs):
                    n = p.numel()
                    full_master[off:off + n].copy_(p.detach().reshape(-1).float())
                    s.model_flat[off:off + n].copy_(p.detach().reshape(-1))
                    p.data = s.model_flat[off:off + n].view(p.shape)
                    p.main_grad = s.grad[off:off + n].view(p.shape)
                s.master = full_master[s.lo:s.lo + per].clone()
                del full_master
                s.gshard = torch.zeros(per, dtype=torch.float32, device=self.device)
            else:
                s.per, s.lo = total, 0
                s.grad = torch.zeros(total, dtype=torch.float32, device=self.device)
                s.master = torch.zeros(total, dtype=torch.float32, device=self.device)
                s.model_flat = None
                for p, off in zip(s.params, offs):
                    n = p.numel()
                    s.master[off:off + n].copy_(p.detach().reshape(-1))
                    p.data = s.master[off:off + n].view(p.shape)
                    p.main_grad = s.grad[off:off + n].view(p.shape)
            s.m, s.v = torch.zeros_like(s.master), torch.zeros_like(s.master)
            s.ema = s.master.clone() if cfg.use_ema else None
            for p in s.params:
                p.register_post_accumulate_grad_hook(self._fold_grad)
        self._sumsq = torch.zeros(1, dtype=torch.float64, device=self.device)
        self._sumsq_local = torch.zeros(1, dtype=torch.float64, device=self.device)
        self.uses_multicast = any(getattr(s, "mc_grad", 0) for s in self.segments)
        self.barrier()

    @staticmethod
    def _fold_grad(p):
        if p.grad is not None:
            p.main_grad.add_(p.grad.float())
            p.grad = None

    def grad_buffers(self):
        return [s.grad for s in self.segments]

    def zero_grad(self):
        for s in self.segments:
            s.grad.zero_()

    def reduce_and_step(self, batch_img: int, grad_scale: float, extra_sumsq: torch.Tensor | None = None) -> torch.Tensor:
        """Whole update. Returns the device scalar with the squared global gradient norm (after scaling).
        ``extra_sumsq``: squared norm (already scaled and complete) of gradients that another optimizer manages and
        that count towards the same clipping norm (tensor-parallel shards)."""
        nsq = self.reduce_scatter(grad_scale)
        if extra_sumsq is not None:
            nsq += extra_sumsq.to(nsq.dtype)
        return self.apply(batch_img, grad_scale, nsq)

    def reduce_scatter(self, grad_scale: float) -> torch.Tensor:
        """First half: every rank's shard of the summed, scaled gradient lands in ``gshard`` and the squared norm of the
        whole reduced gradient (all segments, all ranks of the group) is returned as a device scalar. A caller that
        clips over more than this group (pipeline stages) adds the other parts to it before :meth:`apply`."""
        lib = L.lib()
        f = ctypes.c_float
        self._sumsq.zero_()
        self._sumsq_local.zero_()
        self.barrier()                                   # every rank's backward pass has finished writing gradients
        for s in self.segments:
            if s.low_precision:
                rc = lib.aeris_grad_reduce_scatter(s.grad_ptrs, ctypes.c_void_p(s.mc_grad), self.world,
                                                   ctypes.c_longlong(s.lo), ctypes.c_longlong(s.per), f(grad_scale),
                                                   L.ptr(s.gshard), L.ptr(self._sumsq), L.stream_ptr())
                L.check(rc, "aeris_grad_reduce_scatter")
            else:
                dist.all_reduce(s.grad, group=self.group)
                E.sumsq(s.grad, self._sumsq_local)
        # the scalar reduction doubles as the barrier that says every rank has finished READING peer gradients
        dist.all_reduce(self._sumsq, group=self.group)
        self._sumsq += self._sumsq_local * (grad_scale * grad_scale)
        return self._sumsq

    def apply(self, batch_img: int, grad_scale: float, norm_sq: torch.Tensor) -> torch.Tensor:
        """Second half: clip by ``norm_sq``, AdamW on the master shard, bf16 weights stored into every peer's buffer."""
        c, lib = self.cfg, L.lib()
        f = ctypes.c_float
        self.step_count += 1
        lr = lr_at(self.cur_nimg, c.lr, c)
        beta = ema_beta_at(self.cur_nimg, batch_img, c) if c.use_ema else None
        if norm_sq is not self._sumsq:
            self._sumsq.copy_(norm_sq.to(self._sumsq.dtype).reshape(self._sumsq.shape))
        max_norm = c.grad_clip_max_norm if c.grad_clip else 0.0
        for s in self.segments:
            wd = c.weight_decay if s.decay else 0.0
            eb = beta if (beta is not None and s.ema is not None) else -1.0
            if s.low_precision:
                s.grad.zero_()
                rc = lib.aeris_shard_adamw_allgather(
                    L.ptr(s.master), L.ptr(s.gshard), L.ptr(s.m), L.ptr(s.v), L.ptr(s.ema), s.param_ptrs,
                    ctypes.c_void_p(s.mc_param), self.world, ctypes.c_longlong(s.lo), ctypes.c_longlong(s.per),
                    L.ptr(self._sumsq), f(lr), f(c.betas[0]), f(c.betas[1]), f(c.eps), f(wd), self.step_count,
                    f(max_norm), f(eb), L.stream_ptr())
                L.check(rc, "aeris_shard_adamw_allgather")
            else:
                E.adamw(s.master, s.grad, s.m, s.v, None, s.ema if eb >= 0 else None, self._sumsq, lr=lr,
                        betas=c.betas, eps=c.eps, weight_decay=wd, step=self.step_count, grad_scale=grad_scale,
                        max_norm=max_norm, ema_beta=eb)
        self.barrier()                                   # every peer's stores into my parameter buffer have landed
        self.cur_nimg += batch_img
        self.last_lr = lr
        return self._sumsq

    # ---- state in the layout of FlatOptimizer (collective: every rank of the group calls, all get the full dicts) ------
    host_copies = True      # False on ranks that only take part in the gathers of a checkpoint another rank writes

    def _gather_full(self, s, shard: torch.Tensor) -> torch.Tensor | None:
        if not s.low_precision:
            return shard.detach().cpu().clone() if self.host_copies else None
        full = torch.empty(s.padded, dtype=torch.float32, device=self.device)
        dist.all_gather_into_tensor(full, shard.contiguous(), group=self.group)
        out = full.cpu() if self.host_copies else None
        del full
        return out

    def _named(self, which: str) -> dict[str, torch.Tensor]:
        out = {}
        for s in self.segments:
            shard = getattr(s, which)
            if shard is None:
                continue
            full = self._gather_full(s, shard)
            if full is None:
                continue
            for name, p, off in zip(s.names, s.params, s.offs):
                out[name] = full[off:off + p.numel()].view(p.shape)
        return out

    def master_state_dict(self) -> dict[str, torch.Tensor]:
        return self._named("master")

    def ema_state_dict(self) -> dict[str, torch.Tensor]:
        return self._named("ema")

    def state_dict(self) -> dict:
        return {"step": self.step_count, "cur_nimg": self.cur_nimg, "exp_avg": self._named("m"),
                "exp_avg_sq": self._named("v")}

    def load_state_dict(self, sd: dict, master: dict | None = None, ema: dict | None = None):
        """Inverse of the three dicts above: every rank takes its shard of each array; the bf16 model copy is rebuilt
        from the masters on every rank."""
        self.step_count, self.cur_nimg = int(sd["step"]), int(sd["cur_nimg"])
        sources = {"m": sd.get("exp_avg"), "v": sd.get("exp_avg_sq"), "master": master, "ema": ema}
        for s in self.segments:
            for which, named in sources.items():
                dst = getattr(s, which)
                if named is None or dst is None:
                    continue
                for name, p, off in zip(s.names, s.params, s.offs):
                    if name not in named:
                        continue
                    src = named[name].reshape(-1).float()
                    n = p.numel()
                    if s.low_precision:
                        a, b = max(off, s.lo), min(off + n, s.lo + s.per)      # overlap with this rank's shard
                        if a < b:
                            dst[a - s.lo:b - s.lo].copy_(src[a - off:b - off])
                        if which == "master":
                            s.model_flat[off:off + n].copy_(src.to(s.model_flat.dtype))
                    else:
                        dst[off:off + n].copy_(src)
        self.barrier()

    # ---- per-rank shard state (no communication) ------------------------------------------------------------------
    def shard_state(self) -> dict:
        return {"step": self.step_count, "cur_nimg": self.cur_nimg, "rank": self.rank, "world": self.world,
                "segments": [{"master": s.master.cpu(), "m": s.m.cpu(), "v": s.v.cpu(),
                              "ema": None if s.ema is None else s.ema.cpu()} for s in self.segments]}

    def load_shard_state(self, sd: dict):
        assert sd["world"] == self.world and sd["rank"] == self.rank
        self.step_count, self.cur_nimg = sd["step"], sd["cur_nimg"]
        for s, d in zip(self.segments, sd["segments"]):
            s.master.copy_(d["master"]); s.m.copy_(d["m"]); s.v.copy_(d["v"])
            if s.ema is not None and d["ema"] is not None:
                s.ema.copy_(d["ema"])
