"""Flat-buffer parameter store, gradient accumulation, LR schedule, clipping, AdamW with fp32 masters and EMA.

What the reference does (src/aeris/parallelism/parallel_engine.py): a flat fp32 gradient buffer with per-parameter
``main_grad`` views filled by post-accumulate hooks (:1281-1319); reduce over the weight group, scale by
1/(DP*GAS), global-norm clip with the norm summed over pipeline stages (:709-724); fp32 master weights, the optimizer
and the EMA on the CPU with a full D2H/H2D round trip per step (:727-738, :862-884); piecewise LR schedule
(:799-830). Here everything stays on the GPU: one fused kernel per segment applies scale, clip, NaN guard, AdamW on
the fp32 master, the bf16 weight refresh and the EMA update, and zeroes the gradient.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch
import torch.nn as nn


@dataclass
class OptimConfig:
    lr: float = 2e-4
    betas: tuple[float, float] = (0.85, 0.9)
    eps: float = 1e-8
    weight_decay: float = 0.2
    decay_policy: str = "custom_decay5"   # "all" | "custom_decay" | "custom_decay5" (reference train.py:166-223)
    grad_clip: bool = True
    grad_clip_max_norm: float = 20.0
    total_img: int = 25_000_000
    lr_rampup_img: int = 20_000
    lr_min_factor: float = 0.01
    lr_rampdown_start: int = 100_000_000_000
    lr_rampdown_length: int = 50_000_000
    lr_rampdown_ema_min_ratio: float = 1.0
    ema_halflife_img: int = 100_000
    ema_rampup_ratio: float | None = 0.05
    use_ema: bool = True


def lr_at(cur_nimg: int, base_lr: float, c: OptimConfig) -> float:
    """Piecewise schedule of parallel_engine.py:802-830: min_lr after the ramp-down, linear ramp-down window, linear
    warm-up from min_lr, cosine to min_lr otherwise."""
    min_lr = base_lr * c.lr_min_factor
    if cur_nimg > c.lr_rampdown_start + c.lr_rampdown_length:
        return min_lr
    if cur_nimg > c.lr_rampdown_start:
        prog = 1.0 - (cur_nimg - c.lr_rampdown_start) / c.lr_rampdown_length
        return min_lr + (base_lr - min_lr) * prog
    if cur_nimg < c.lr_rampup_img:
        return min_lr + (base_lr - min_lr) * (cur_nimg / c.lr_rampup_img)
    prog = min(1.0, (cur_nimg - c.lr_rampup_img) / max(c.total_img - c.lr_rampup_img, 1))
    return min_lr + 0.5 * (base_lr - min_lr) * (1 + math.cos(math.pi * prog))


def ema_beta_at(cur_nimg: int, batch_img: int, c: OptimConfig) -> float | None:
    """EMA coefficient of parallel_engine.py:868-884 (half-life in images with ramp-up and optional ramp-down);
    None once the LR ramp-down has finished (the reference stops updating the EMA there)."""
    if cur_nimg >= c.lr_rampdown_start + c.lr_rampdown_length:
        return None
    hl = c.ema_halflife_img
    if c.ema_rampup_ratio is not None:
        hl = min(hl, cur_nimg * c.ema_rampup_ratio)
    if cur_nimg > c.lr_rampdown_start:
        prog = 1.0 - (cur_nimg - c.lr_rampdown_start) / c.lr_rampdown_length
        mn = c.ema_halflife_img * c.lr_rampdown_ema_min_ratio
        hl = mn + (c.ema_halflife_img - mn) * prog
    return 0.5 ** (batch_img / max(hl, 1e-8))


def no_decay_names(model: nn.Module, policy: str) -> set[str]:
    """Parameter names excluded from weight decay. ``custom_decay5`` reproduces the reference's observable behaviour
    (train.py:178-183 tests ``isinstance(param, nn.Linear)`` on parameters, so every parameter lands in the
    no-decay group); ``custom_decay`` follows train.py:205-210 (no decay for ``proj``, ``head`` and non-modulation
    ``norm`` parameters); ``all`` decays everything."""
    names = [n for n, p in model.named_parameters() if p.requires_grad]
    if policy == "custom_decay5":
        return set(names)
    if policy == "custom_decay":
        return {n for n in names if "proj" in n or "head" in n or ("norm" in n and "modulation" not in n)}
    return set()


@dataclass
class _Segment:
    name: str
    params: list = field(default_factory=list)
    names: list = field(default_factory=list)
    decay: bool = True
    low_precision: bool = True
    numel: int = 0
    master: torch.Tensor | None = None
    grad: torch.Tensor | None = None
    m: torch.Tensor | None = None
    v: torch.Tensor | None = None
    ema: torch.Tensor | None = None
    model_flat: torch.Tensor | None = None   # bf16 flat buffer the module parameters view (low_precision only)


class FlatOptimizer:
    """Owns flat fp32 master / gradient / Adam state / EMA buffers; module parameters become views of flat buffers.

    Segments: {bf16-parameter, fp32-parameter} x {decay, no-decay}. Parameters that take part in the fused block
    backward get ``param.main_grad`` (fp32 view) which the weight-gradient GEMM epilogue accumulates into; every
    other parameter gets a post-accumulate hook that folds ``.grad`` into ``main_grad`` and frees it.
    """

    def __init__(self, model: nn.Module, cfg: OptimConfig, device=None, params=None):
        """``params``: the (name, parameter) pairs to manage; default: every trainable parameter of ``model``."""
        self.cfg = cfg
        self.model = model
        self.step_count = 0
        self.cur_nimg = 0
        nd = no_decay_names(model, cfg.decay_policy)
        segs: dict[tuple[bool, bool], _Segment] = {}
        for n, p in (params if params is not None else model.named_parameters()):
            if not p.requires_grad:
                continue
            key = (p.dtype != torch.float32, n not in nd)
            seg = segs.setdefault(key, _Segment(name=f"{'lp' if key[0] else 'fp32'}_{'decay' if key[1] else 'nodecay'}",
                                                decay=key[1], low_precision=key[0]))
            seg.params.append(p)
            seg.names.append(n)
        self.segments = list(segs.values())
        self._hooks = []
        for seg in self.segments:
            dev = device or seg.params[0].device
            # 16-element alignment of every parameter inside the flat buffers keeps vector accesses and TMA legal
            offs, total = [], 0
            for p in seg.params:
                offs.append(total)
                total += (p.numel() + 15) // 16 * 16
            seg.numel = total
            seg.master = torch.zeros(total, dtype=torch.float32, device=dev)
            seg.grad = torch.zeros(total, dtype=torch.float32, device=dev)
            seg.m = torch.zeros(total, dtype=torch.float32, device=dev)
            seg.v = torch.zeros(total, dtype=torch.float32, device=dev)
            if seg.low_precision:
                seg.model_flat = torch.zeros(total, dtype=seg.params[0].dtype, device=dev)
            for p, off in zip(seg.params, offs):
                n = p.numel()
                seg.master[off:off + n].copy_(p.detach().reshape(-1).float())
                target = seg.model_flat if seg.low_precision else seg.master
                if seg.low_precision:
                    target[off:off + n].copy_(p.detach().reshape(-1))
                p.data = target[off:off + n].view(p.shape)
                p.main_grad = seg.grad[off:off + n].view(p.shape)
                self._hooks.append(p.register_post_accumulate_grad_hook(self._fold_grad))
            seg.ema = seg.master.clone() if cfg.use_ema else None
        self._norm_sq = None

    @staticmethod
    def _fold_grad(p: torch.Tensor):
        if p.grad is not None:
            p.main_grad.add_(p.grad.float())
            p.grad = None

    def grad_buffers(self) -> list[torch.Tensor]:
        return [s.grad for s in self.segments]

    def zero_grad(self):
        for s in self.segments:
            s.grad.zero_()

    def grad_norm_sq(self, grad_scale: float) -> torch.Tensor:
        """Device scalar (float64): sum of squares of (grad * grad_scale) over this rank's buffers."""
        dev = self.segments[0].grad.device if self.segments else "cpu"
        if self._norm_sq is None:
            self._norm_sq = torch.zeros(1, dtype=torch.float64, device=dev)
        self._norm_sq.zero_()
        if dev.type == "cuda":
            from ..ops import elementwise as E
            for s in self.segments:
                E.sumsq(s.grad, self._norm_sq)
        else:
            for s in self.segments:
                self._norm_sq += s.grad.double().pow(2).sum()
        self._norm_sq *= grad_scale * grad_scale
        return self._norm_sq

    def step(self, batch_img: int, grad_scale: float, norm_sq: torch.Tensor | None = None):
        """One optimizer step. ``grad_scale`` multiplies the accumulated gradient (1 / (DP * GAS));
        ``norm_sq`` is the global squared norm of the scaled gradient (already reduced over ranks/stages)."""
        c = self.cfg
        self.step_count += 1
        lr = lr_at(self.cur_nimg, c.lr, c)
        beta = ema_beta_at(self.cur_nimg, batch_img, c) if c.use_ema else None
        max_norm = c.grad_clip_max_norm if (c.grad_clip and norm_sq is not None) else 0.0
        for s in self.segments:
            wd = c.weight_decay if s.decay else 0.0
            if s.master.is_cuda:
                from ..ops import elementwise as E
                E.adamw(s.master, s.grad, s.m, s.v, s.model_flat, s.ema if beta is not None else None, norm_sq,
                        lr=lr, betas=c.betas, eps=c.eps, weight_decay=wd, step=self.step_count,
                        grad_scale=grad_scale, max_norm=max_norm, ema_beta=beta if beta is not None else -1.0)
            else:
                self._step_cpu(s, lr, wd, grad_scale, max_norm, norm_sq, beta)
        self.cur_nimg += batch_img
        self.last_lr = lr

    def _step_cpu(self, s: _Segment, lr, wd, grad_scale, max_norm, norm_sq, beta):
        c = self.cfg
        clip = 1.0
        if max_norm > 0 and norm_sq is not None:
            cc = max_norm / (float(norm_sq.sqrt()) + 1e-6)
            clip = min(1.0, cc)
        g = torch.nan_to_num(s.grad * (grad_scale * clip), nan=0.0, posinf=1e5, neginf=-1e5)
        b1, b2 = c.betas
        s.m.mul_(b1).add_(g, alpha=1 - b1)
        s.v.mul_(b2).addcmul_(g, g, value=1 - b2)
        s.master.mul_(1 - lr * wd)
        denom = (s.v / (1 - b2 ** self.step_count)).sqrt_().add_(c.eps)
        s.master.addcdiv_(s.m / (1 - b1 ** self.step_count), denom, value=-lr)
        if s.model_flat is not None:
            s.model_flat.copy_(s.master)
        if s.ema is not None and beta is not None:
            s.ema.copy_(s.master.lerp(s.ema, beta))
        s.grad.zero_()

    # ---- state for checkpoints -------------------------------------------------------------------------------
    def _named_views(self, which: str) -> dict[str, torch.Tensor]:
        out = {}
        for s in self.segments:
            buf = getattr(s, which)
            if buf is None:
                continue
            off = 0
            for n, p in zip(s.names, s.params):
                out[n] = buf[off:off + p.numel()].view(p.shape)
                off += (p.numel() + 15) // 16 * 16
        return out

    def master_state_dict(self) -> dict[str, torch.Tensor]:
        return self._named_views("master")

    def ema_state_dict(self) -> dict[str, torch.Tensor]:
        return self._named_views("ema")

    def state_dict(self) -> dict:
        return {"step": self.step_count, "cur_nimg": self.cur_nimg,
                "exp_avg": {k: v.clone() for k, v in self._named_views("m").items()},
                "exp_avg_sq": {k: v.clone() for k, v in self._named_views("v").items()}}

    def load_state_dict(self, sd: dict, master: dict | None = None, ema: dict | None = None):
        self.step_count, self.cur_nimg = sd["step"], sd["cur_nimg"]
        for which, src in (("m", sd["exp_avg"]), ("v", sd["exp_avg_sq"]), ("master", master), ("ema", ema)):
            if src is None:
                continue
            views = self._named_views(which)
            for k, v in views.items():
                if k in src:
                    v.copy_(src[k])
        if master is not None:
            for s in self.segments:
                if s.model_flat is not None:
                    s.model_flat.copy_(s.master)
