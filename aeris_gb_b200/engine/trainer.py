"""Single-node training engine: window-parallel (WP) x data-parallel TrigFlow training with every logical pipeline
stage resident on each GPU (one process per GPU, NCCL for plumbing, peer-memory kernels for the halo exchange).

Public API::

    trainer = Trainer(model_cfg, optim_cfg, diff_cfg, device)       # after torch.distributed is initialised (or not)
    loss = trainer.train_step(target_host, cond_host)               # pinned host tensors in, python float out

What it replaces in the reference: ``ParallelEngine.exec_schedule`` with load -> fwd -> bwd -> reduce -> step
(src/aeris/parallelism/parallel_engine.py:585-686, 889-1017, 696-887) for the case PP = 1 (all stages local), with
the per-rank data tiles of ``scripts/data_processing/wp_create.py`` replaced by contiguous image blocks.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.distributed as dist
import torch.utils.checkpoint as ckpt

from ..diffusion import trigflow as TF
from ..models import layout as LY
from ..models.aeris import AerisConfig, AerisModel, StreamContext
from .optim import FlatOptimizer, OptimConfig


@dataclass
class DiffusionConfig:
    sigma_data: float = 1.0
    sigma_min: float = 0.2
    sigma_max: float = 500.0
    w_lat_add: float = 0.01
    noise_law: str = "loguniform"
    cond_channels: int = 74
    grad_scale_parity: bool = True   # reference sums local-mean gradients over WP ranks without dividing by WP


def wp_grid_for(n: int) -> tuple[int, int]:
    return {1: (1, 1), 2: (1, 2), 4: (2, 2), 8: (2, 4), 16: (4, 4)}[n]


class Trainer:
    def __init__(self, model_cfg: AerisConfig, optim_cfg: OptimConfig, diff_cfg: DiffusionConfig, device,
                 seed: int = 1234, wp_group=None, dp_size: int = 1, dp_rank: int = 0, model: AerisModel | None = None,
                 fused_dp: bool | None = None, use_multicast: bool = False, sp_group=None,
                 fused_io: bool | None = None, weight_group=None, tp_group=None, tp_ortho_group=None):
        self.cfg, self.ocfg, self.dcfg = model_cfg, optim_cfg, diff_cfg
        self.device = torch.device(device)
        # `wp_group`: every rank that shares a sample (WP grid x SP), ordered (wp_y, wp_x, sp); `sp_group`: the ranks that
        # share this rank's windows (Ulysses)
        self.wp_group = wp_group
        self.sp_group = sp_group
        # `weight_group`: every rank that holds a replica of the weights (WP x SP x DP); gradients are reduced over it
        self.weight_group = weight_group if weight_group is not None else wp_group
        # `tp_group` (model_cfg.tp > 1): the ranks that split the MLP weights between them; they hold different token
        # rows of the same sample. Default: the SP group when sp > 1, else the WP group. `tp_ortho_group`: the ranks of
        # the weight group that hold the same shard (None when the tensor-parallel group is the whole weight group)
        self.tp_group = None
        if model_cfg.tp > 1:
            self.tp_group = tp_group if tp_group is not None else (sp_group if model_cfg.sp > 1 else wp_group)
            assert self.tp_group is not None and dist.get_world_size(self.tp_group) == model_cfg.tp, \
                "AerisConfig.tp must equal the size of the tensor-parallel group"
            assert model_cfg.tp_rank == dist.get_rank(self.tp_group), "AerisConfig.tp_rank is this rank's place in it"
            n_weight = dist.get_world_size(self.weight_group) if self.weight_group is not None else 1
            assert tp_ortho_group is not None or n_weight == model_cfg.tp, \
                "a weight group larger than the tensor-parallel group needs tp_ortho_group"
        self.wp_size = model_cfg.wp[0] * model_cfg.wp[1] * model_cfg.sp
        self.wp_rank = dist.get_rank(wp_group) if (self.wp_size > 1) else 0
        self.sp_rank = self.wp_rank % model_cfg.sp
        self.dp_size, self.dp_rank = dp_size, dp_rank
        torch.manual_seed(seed)   # identical initial weights on every rank
        self.model = (model or AerisModel(model_cfg)).to(self.device)
        # weight-group collectives: this library's peer-memory kernels (default on GPUs with > 1 rank) or NCCL
        n_replicas = self.wp_size * dp_size
        self.fused_dp = (n_replicas > 1 and self.device.type == "cuda") if fused_dp is None else fused_dp
        if self.tp_group is not None:
            from .tp_optim import TPOptimizer
            self.opt = TPOptimizer(self.model, optim_cfg, self.device, self.weight_group, self.tp_group, tp_ortho_group,
                                   fused=self.fused_dp, use_multicast=use_multicast)
        elif self.fused_dp:
            from .fused_dp import FusedShardedOptimizer
            self.opt = FusedShardedOptimizer(self.model, optim_cfg, self.weight_group, self.device, use_multicast)
        else:
            self.opt = FlatOptimizer(self.model, optim_cfg)
        self.grid = model_cfg.grid()
        # noise: one stream per (wp rank, dp rank); noise level: one per dp replica, shared by its WP ranks
        # (parallel_engine.py:119-120)
        self.rng = torch.Generator(device=self.device)
        self.rng.manual_seed(seed + 1000 * dp_rank + self.wp_rank)
        self.nl_rng = torch.Generator(device=self.device)
        self.nl_rng.manual_seed(seed + dp_rank)
        self._ctx: dict[int, StreamContext] = {}
        self._w_lat_tok = None
        self._w_var = TF.variable_weights(model_cfg.out_channels, self.device)
        self.halo = None
        if self.wp_size > 1:
            from ..parallel.symm import HaloExchange
            self.halo = HaloExchange(wp_group, self.device)
        # noising, embedding, output head and loss on this library's kernels (counter-based noise that does not depend
        # on the WP/SP layout) or, with fused_io=False, the PyTorch formulation with torch.randn noise
        self.fused_io = (self.device.type == "cuda") if fused_io is None else fused_io
        self.seed = seed
        self.step_count = 0
        self._io_tables = None
        # device timers / NVTX ranges around the phases of a step (resolved lazily; enable with trainer.timers.enabled)
        from ..utils.timers import DeviceTimers
        self.timers = DeviceTimers(enabled=False)
        if self.halo is not None:
            self.halo.timers = self.timers
        self.last_norm = 0.0
        self._sp_exchange = None
        self._tp_exchange = None

    # ------------------------------------------------------------------------------------------------ helpers
    def context(self, batch: int) -> StreamContext:
        if batch not in self._ctx:
            peer_fn = self.halo.peer_fn if self.halo is not None else None
            ctx = StreamContext(self.cfg, batch, self.wp_rank, peer_fn, wp_group=self.wp_group, sp_group=self.sp_group,
                                tp_group=self.tp_group)
            if self.tp_group is not None and self.device.type == "cuda":
                if self._tp_exchange is None:
                    from ..parallel.tensor import TPExchange
                    self._tp_exchange = TPExchange(self.tp_group, self.device)
                ctx.tp_exchange = self._tp_exchange
            if self.cfg.sp > 1 and self.device.type == "cuda":
                if self._sp_exchange is None:
                    from ..models.fused import SPExchange
                    self._sp_exchange = SPExchange(self.sp_group, self.device)
                ctx.sp_exchange = self._sp_exchange
            self._ctx[batch] = ctx
        return self._ctx[batch]

    def w_lat_tokens(self) -> torch.Tensor:
        if self._w_lat_tok is None:
            w = TF.latitude_weights(self.cfg.img[0], self.dcfg.w_lat_add)
            img = w.view(1, -1, 1, 1).expand(1, self.cfg.img[0], self.cfg.img[1], 1)
            self._w_lat_tok = LY.image_to_tokens(img, self.grid, (0, 0), self.wp_rank).to(self.device)
        return self._w_lat_tok

    def block_to_tokens(self, block: torch.Tensor) -> torch.Tensor:
        """[B, H/wp_y, W/wp_x, C] block of this rank -> [B * tokens_per_rank, C] rows of the unshifted layout."""
        B, hb, wb, C = block.shape
        g = self.grid
        x = block.view(B, g.nwy_loc, g.ws_y, g.nwx_loc, g.ws_x, C).permute(0, 1, 3, 2, 4, 5)
        x = x.reshape(B * g.windows_per_rank, g.L, C)
        if g.sp > 1:      # this rank's contiguous slice of every window's token sequence
            x = x[:, self.sp_rank * g.n_local:(self.sp_rank + 1) * g.n_local]
        return x.reshape(B * g.tokens_per_rank, C)

    def tokens_to_block(self, tok: torch.Tensor, B: int) -> torch.Tensor:
        g = self.grid
        C = tok.shape[-1]
        x = tok.view(B, g.nwy_loc, g.nwx_loc, g.ws_y, g.ws_x, C).permute(0, 1, 3, 2, 4, 5)
        return x.reshape(B, g.nwy_loc * g.ws_y, g.nwx_loc * g.ws_x, C)

    # ------------------------------------------------------------------------------------------------ training
    def loss_tokens(self, x_tok: torch.Tensor, cond_tok: torch.Tensor, t: torch.Tensor, z: torch.Tensor) -> torch.Tensor:
        """Sum over the local batch of the per-sample local-token-mean TrigFlow losses."""
        B = t.shape[0]
        rows = x_tok.shape[0] // B
        ctx = self.context(B)
        sd = self.dcfg.sigma_data
        tr = t.repeat_interleave(rows)
        model_in = TF.noise_inputs(x_tok, cond_tok, z, tr, sd)
        pred = self.model.forward_tokens(model_in, t, ctx)
        w_lat = self.w_lat_tokens().repeat(B, 1)
        err = (sd * pred - TF.v_target(x_tok, z, tr)) ** 2 * self._w_var * w_lat
        return err.sum(dim=-1).view(B, rows).mean(dim=1).sum()

    def loss_regression(self, in_tok: torch.Tensor, target_tok: torch.Tensor, interval: torch.Tensor | None) -> torch.Tensor:
        """Non-diffusion modes (``rit`` / plain): weighted squared error of the model's output against the target
        state, mean over the local tokens, summed over the local batch (parallel_engine.py:998)."""
        B = in_tok.shape[0] // self.grid.tokens_per_rank
        rows = in_tok.shape[0] // B
        pred = self.model.forward_tokens(in_tok, interval, self.context(B))
        w_lat = self.w_lat_tokens().repeat(B, 1)
        err = (pred - target_tok) ** 2 * self._w_var * w_lat
        return err.sum(dim=-1).view(B, rows).mean(dim=1).sum()

    def io_plan(self, batch: int, noise: bool = True, seed: int | None = None):
        from ..models import fused_io
        from ..ops import diffusion as DF
        if self._io_tables is None:
            ay, ax = fused_io.ape_tables(self.cfg, self.device)
            w_lat = TF.latitude_weights(self.cfg.img[0], self.dcfg.w_lat_add).to(self.device).contiguous()
            self._io_tables = (ay, ax, w_lat)
        ay, ax, w_lat = self._io_tables
        geom = DF.make_geom(self.grid, batch, self.wp_rank, sample0=self.dp_rank * batch)
        if seed is None:
            seed = (self.seed << 32) + self.step_count
        return fused_io.IoPlan(geom, self.dcfg.sigma_data, seed, noise, ay, ax, self._w_var, w_lat,
                               self.cfg.eps(self.cfg.data_dtype))

    def loss_images(self, x: torch.Tensor, c: torch.Tensor, t: torch.Tensor, seed: int | None = None) -> torch.Tensor:
        """Fused-kernel counterpart of :meth:`loss_tokens`: x [B, hb, wb, C_out], c [B, hb, wb, C_cond] on the device."""
        B = x.shape[0]
        cs = torch.stack([torch.cos(t), torch.sin(t)], dim=1).float().contiguous()
        return self.model.loss_images(x.contiguous(), c.contiguous(), cs, t, self.context(B), self.io_plan(B, seed=seed))

    def train_step(self, target_host: torch.Tensor, cond_host: torch.Tensor, read_loss: bool = True,
                   interval: torch.Tensor | None = None):
        """One optimizer step on this rank's blocks of ``B`` samples. target_host: [B, H/wp_y, W/wp_x, C_out] fp32
        (standardised residual), cond_host: [B, H/wp_y, W/wp_x, C_cond] fp32; both pinned host tensors.
        Non-diffusion modes: ``cond_host`` is the model input, ``target_host`` the state to predict and ``interval``
        [B] the forecast interval (rit). Returns the loss averaged over the local batch (synchronises: the value is
        read back to the host)."""
        dev = self.device
        with self.timers.region("load"):
            x = target_host.to(dev, non_blocking=True)
            c = cond_host.to(dev, non_blocking=True)
            B = x.shape[0]
            if self.cfg.diffusion:
                t = TF.sample_noise_level(B, self.dcfg.sigma_min, self.dcfg.sigma_max, self.dcfg.sigma_data,
                                          generator=self.nl_rng, device=dev, law=self.dcfg.noise_law)
        with self.timers.region("fwd"):
            if not self.cfg.diffusion:
                iv = interval.to(dev).float() if interval is not None else None
                loss = self.loss_regression(self.block_to_tokens(c), self.block_to_tokens(x), iv)
            elif self.fused_io:
                loss = self.loss_images(x, c, t)
            else:
                x_tok, c_tok = self.block_to_tokens(x), self.block_to_tokens(c)
                z = torch.randn(x_tok.shape, generator=self.rng, device=dev) * self.dcfg.sigma_data
                loss = self.loss_tokens(x_tok, c_tok, t, z)
        with self.timers.region("bwd"):
            loss.backward()
        if read_loss:
            # a bounded device wait that ran out (a peer that never signalled) leaves incomplete activations or
            # gradients behind: raise before the optimizer applies them and the all-gather spreads them
            try:
                self.check_device()
            except Exception:
                for buf in self.opt.grad_buffers():
                    buf.zero_()
                raise
        with self.timers.region("reduce_step"):
            self.reduce_and_step(B)
        self.step_count += 1
        self.last_loss = loss.detach()
        if not read_loss:
            return None
        value = float(self.last_loss.item()) / B
        self.check_device()
        return value

    def resume(self, cur_nimg: int, gas: int = 1) -> None:
        """After a checkpoint load: continue the step counter (it seeds the counter-based noise of the fused input
        kernels) and the noise / noise-level generators where a run of ``cur_nimg`` images would be, instead of
        replaying the draws of step 0 (parallel_engine.py:1155-1156)."""
        self.step_count = cur_nimg // max(1, gas * self.dp_size)
        self.rng.manual_seed(self.seed + 1000 * self.dp_rank + self.wp_rank + cur_nimg)
        self.nl_rng.manual_seed(self.seed + self.dp_rank + cur_nimg)

    def check_device(self) -> None:
        """Raise ``KernelError`` if a kernel of this library recorded a device-side error (time-out of a bounded wait,
        failed bounds check) since the last check. Reads one word from the device, so it synchronises."""
        if self.device.type == "cuda":
            from ..ops import lib as L
            L.check_status(sync=False)

    def reduce_and_step(self, local_batch: int):
        gas = local_batch
        scale = 1.0 / (self.dp_size * gas)
        if not self.dcfg.grad_scale_parity:
            scale /= self.wp_size
        if self.fused_dp or self.tp_group is not None:
            self._nsq = self.opt.reduce_and_step(gas * self.dp_size, scale)
            return
        if self.wp_size > 1 or self.dp_size > 1:
            for buf in self.opt.grad_buffers():
                dist.all_reduce(buf, group=self.weight_group)
        nsq = self.opt.grad_norm_sq(scale) if self.ocfg.grad_clip else None
        self.opt.step(batch_img=gas * self.dp_size, grad_scale=scale, norm_sq=nsq)
        self._nsq = nsq

    def grad_norm(self) -> float:
        return float(self._nsq.sqrt().item()) if getattr(self, "_nsq", None) is not None else 0.0

    # ------------------------------------------------------------------------------------------------ metrics
    def flops_per_step(self, global_batch: int) -> float:
        return self.cfg.flops_per_sample() * global_batch
