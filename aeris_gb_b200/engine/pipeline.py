"""Pipeline-parallel training engine: PP x WP x SP x DP with an instruction interpreter over the schedules of
:mod:`aeris_gb_b200.parallel.schedule`.

Counterpart of the reference's ``ParallelEngine`` (src/aeris/parallelism/parallel_engine.py): rank grid and groups
(:294-451), pipe buffers (:1246-1279), micro-batch load with TrigFlow noising on the first stage and targets on the last
(:585-686), forward / backward per micro-batch with received activations turned into leaves (:889-1017, :1070-1075),
p2p send/recv of activations and gradients (:1019-1116), gradient reduction over the weight group with the global norm
summed over pipeline stages (:696-792), optimizer step + EMA (:794-887), per-stage checkpoints (:1119-1160), warm-up
straggler probe (:1492-1533) and per-instruction timers (:1202-1223).

Differences by design: any SP / WP / PP that divides the model (the reference asserts SP == 12); a physical pipeline
rank may hold several logical stages; the half-window shift is a table-driven re-partition inside the stage (peer
memory on GPUs); master weights, optimizer and EMA stay on the device; no host synchronisation per micro-batch (the
loss is accumulated on the device); pipeline p2p is NCCL (gloo on CPU) on the rank pairs of the PP group.
"""
from __future__ import annotations

import os
import time
from dataclasses import dataclass, field

import torch
import torch.distributed as dist

from ..diffusion import trigflow as TF
from ..models import layout as LY
from ..models.aeris import AerisConfig, StreamContext
from ..models.stages import PipelineStage, split_stages
from ..parallel import schedule as SCH
from ..parallel.topology import ProcessGrid
from .checkpoint import load_stage_checkpoint, save_stage_checkpoint
from .init import init_params
from .optim import FlatOptimizer, OptimConfig
from .p2p import PipeLinks
from .trainer import DiffusionConfig


@dataclass
class EngineConfig:
    gas: int = 1                          # micro-batches per optimizer step (batch 1 each, as in the reference)
    overlap_p2p: bool = False
    dist_optimizer: bool = False
    fused_io: bool | None = None      # noising + embedding and head + loss on the CUDA kernels (default: on GPUs)
    rs_grads: bool = True
    checkpoint_dir: str | None = None
    checkpoint_every: int = 100           # iterations (:1225)
    checkpoint_keep_every: int = 1000     # extra numbered copy (:1124)
    init_policy: dict = field(default_factory=dict)
    benchmark: bool = False
    seed: int = 0


class ParallelEngine:
    def __init__(self, model_cfg: AerisConfig, optim_cfg: OptimConfig, diff_cfg: DiffusionConfig, ecfg: EngineConfig,
                 grid: ProcessGrid, rank: int, device, data_fn=None, groups: dict | None = None):
        self.cfg, self.ocfg, self.dcfg, self.ecfg = model_cfg, optim_cfg, diff_cfg, ecfg
        self.grid, self.rank, self.device = grid, rank, torch.device(device)
        self.c = grid.coords(rank)
        kinds = ("sp", "pp", "wp", "dp", "weight", "replica", "pipe") + (("tp", "tp_ortho") if model_cfg.tp > 1 else ())
        self.groups = groups if groups is not None else grid.build_groups(rank, kinds=kinds)
        if model_cfg.tp > 1:            # MLP weights split over the SP group (or the WP group) of this stage
            tp_ranks = grid.tp_ranks(rank)
            assert model_cfg.tp == len(tp_ranks), \
                f"model.TP = {model_cfg.tp} must equal the size of the tensor-parallel group ({len(tp_ranks)})"
            model_cfg.tp_rank = tp_ranks.index(rank)
        self.PP, self.GAS = grid.PP, ecfg.gas
        assert (model_cfg.wp[0], model_cfg.wp[1], model_cfg.sp) == (grid.WP_Y, grid.WP_X, grid.SP)
        self.wp_rank = self.c.wp_y * grid.WP_X + self.c.wp_x
        self.replica_rank = self.wp_rank * grid.SP + self.c.sp     # rank inside the WP x SP group holding one sample
        n_logical = model_cfg.n_layers + 2
        self.stage_ids = split_stages(n_logical, self.PP)[self.c.pp]
        torch.manual_seed(ecfg.seed + 17 * self.c.pp)
        self.module = PipelineStage(model_cfg, self.stage_ids).to(self.device)
        init_params(self.module, model_cfg, ecfg.init_policy)
        self._broadcast_params()
        if model_cfg.tp > 1:
            from .tp_optim import TPOptimizer
            assert not ecfg.dist_optimizer, "the sharded NCCL optimizer is not combined with tensor-parallel shards"
            self.opt = TPOptimizer(self.module, optim_cfg, self.device, self.groups.get("weight"), self.groups["tp"],
                                   self.groups.get("tp_ortho"))
        elif ecfg.dist_optimizer and self.device.type == "cuda" and self.groups.get("weight") is not None:
            # the sharded optimizer on this library's peer-memory kernels (reduce-scatter, clip, AdamW and the
            # all-gather of the bf16 weights in two launches per segment); NCCL / gloo ranks take the class below
            from .fused_dp import FusedShardedOptimizer
            self.opt = FusedShardedOptimizer(self.module, optim_cfg, self.groups["weight"], self.device, False)
        elif ecfg.dist_optimizer:
            from .dist_optim import DistOptimizer
            self.opt = DistOptimizer(self.module, optim_cfg, self.groups.get("weight"), rs_grads=ecfg.rs_grads)
        else:
            self.opt = FlatOptimizer(self.module, optim_cfg)
        # The overlapped schedule posts receives a step early and sends right after compute (NCCL and gloo alike:
        # the links have one communicator per direction, see engine/p2p.py).
        sched_cls = SCH.OverlappedTrainSchedule if ecfg.overlap_p2p else SCH.TrainSchedule
        self.schedule = sched_cls(self.GAS, self.PP, self.c.pp)
        nb = self.schedule.num_pipe_buffers()
        self.buf = {k: [None] * nb for k in ("inputs", "outputs", "dt_in", "dt_out", "x", "z", "t", "grad_x", "grad_dt")}
        self.prev_rank = grid.rank_of(self.c.dp, self.c.wp_y, self.c.wp_x, self.c.pp - 1, self.c.sp) if self.c.pp > 0 else None
        self.next_rank = grid.rank_of(self.c.dp, self.c.wp_y, self.c.wp_x, self.c.pp + 1, self.c.sp) if self.c.pp < self.PP - 1 else None
        self.links = PipeLinks(self.groups, self.prev_rank, self.next_rank, self.device)
        if self.PP > 1:
            self.links.warm()
        # the conditioning vector is trainable upstream when one embedding network on the first stage feeds every
        # stage: the shared noise-level MLP (layerwise_t_emb off) or the interval embedding (rit)
        self.dt_grad = self.PP > 1 and model_cfg.conditioned and (model_cfg.rit and not model_cfg.diffusion
                                                                  or not model_cfg.layerwise_t_emb)
        # noise: per (wp, dp, sp), NOT per pp, so the first and last stage regenerate identical z without talking
        # (:119, :667); noise level: per dp replica (:120)
        base = ecfg.seed
        self._noise_seed = base + self.c.wp_x * grid.WP_Y * grid.DP * grid.SP + self.c.wp_y * grid.DP * grid.SP + \
            self.c.dp * grid.SP + self.c.sp
        self.rng = torch.Generator(device=self.device).manual_seed(self._noise_seed)
        self.nl_rng = torch.Generator(device=self.device).manual_seed(base + self.c.dp)
        self.data_fn = data_fn
        self.noise_fn = None
        self.t_fn = None               # tests: noise level as a function of the sample, independent of the DP split
        self.keep_grads = False        # tests: keep a copy of the reduced, scaled gradients of the last step
        self.loads = 0
        self.fused_io = (self.device.type == "cuda" and model_cfg.diffusion) if ecfg.fused_io is None else ecfg.fused_io
        self._io_tables = None
        halo = None
        if grid.WP_Y * grid.WP_X * grid.SP > 1 and self.device.type == "cuda":
            from ..parallel.symm import HaloExchange
            halo = HaloExchange(self.groups["replica"], self.device, pool_gradients=False)
        self.ctx = StreamContext(model_cfg, 1, self.replica_rank, halo.peer_fn if halo else None,
                                 wp_group=self.groups.get("replica"), sp_group=self.groups.get("sp"),
                                 tp_group=self.groups.get("tp"))
        if model_cfg.tp > 1 and self.device.type == "cuda":
            from ..parallel.tensor import TPExchange
            self.ctx.tp_exchange = TPExchange(self.groups["tp"], self.device)
        if grid.SP > 1 and self.device.type == "cuda":
            from ..models.fused import SPExchange
            self.ctx.sp_exchange = SPExchange(self.groups["sp"], self.device)
        self.tokens = self.ctx.grid.tokens_per_rank
        self._w_var = TF.variable_weights(model_cfg.out_channels, self.device)
        w = TF.latitude_weights(model_cfg.img[0], diff_cfg.w_lat_add)
        img = w.view(1, -1, 1, 1).expand(1, model_cfg.img[0], model_cfg.img[1], 1)
        self._w_lat = LY.image_to_tokens(img, self.ctx.grid, (0, 0), self.replica_rank).to(self.device)
        self.loss_acc = torch.zeros((), device=self.device)
        self.tot_loss, self.total_norm, self.stage_norm = 0.0, 0.0, 0.0
        self.cur_it = 0
        self._pending = {}
        self.timers: dict[str, float] = {}
        self._imap = {
            SCH.LoadMicroBatch: self.load, SCH.ForwardPass: self.fwd, SCH.BackwardPass: self.bwd,
            SCH.SendActivation: self.send, SCH.RecvActivation: self.recv, SCH.SendGrad: self.send_grad,
            SCH.RecvGrad: self.recv_grad, SCH.SubmitRecvActivation: self.submit_recv,
            SCH.SubmitRecvGrad: self.submit_recv_grad, SCH.ProcessActivation: self.process_recv,
            SCH.ProcessGrad: self.process_grad, SCH.ReduceTiedGrads: self.placeholder,
            SCH.ReduceGrads: self.reduce_grads, SCH.OptimizerStep: self.step,
        }

    # ------------------------------------------------------------------------------------------------ helpers
    @property
    def cur_nimg(self) -> int:
        return self.opt.cur_nimg

    def is_first_stage(self) -> bool:
        return self.c.pp == 0

    def is_last_stage(self) -> bool:
        return self.c.pp == self.PP - 1

    def placeholder(self, buffer_id=None):
        pass

    def _broadcast_params(self):
        g = self.groups.get("weight")
        if g is None:
            return
        src = self.grid.rank_of(0, 0, 0, self.c.pp, 0)
        from ..parallel.tensor import tp_kind
        ortho = self.groups.get("tp_ortho")
        for n, p in self.module.named_parameters():
            if self.cfg.tp > 1 and tp_kind(n, p) is not None:
                if ortho is not None:        # a shard is shared by the ranks that hold the same one
                    dist.broadcast(p.data, src=self.grid.tp_ortho_ranks(self.rank)[0], group=ortho)
                continue
            dist.broadcast(p.data, src=src, group=g)

    def _sp_slice(self, tok: torch.Tensor) -> torch.Tensor:
        """This SP rank's contiguous slice of every window's tokens. tok: [windows * L, C] (whole windows)."""
        SP = self.grid.SP
        if SP == 1:
            return tok
        L = self.ctx.grid.L
        n = L // SP
        return tok.view(-1, L, tok.shape[-1])[:, self.c.sp * n:(self.c.sp + 1) * n].reshape(-1, tok.shape[-1])

    def _io_plan(self):
        """What the fused input and output ends need for the micro-batch about to be loaded. The noise is counter
        based: seed = (engine seed, optimizer step), counter = (global sample index, pixel, channel), so the first and
        the last pipeline stage draw the same field without talking, whatever the WP / SP / PP split."""
        from ..models import fused_io
        from ..ops import diffusion as DF
        if self._io_tables is None:
            ay, ax = fused_io.ape_tables(self.cfg, self.device)
            w_lat = TF.latitude_weights(self.cfg.img[0], self.dcfg.w_lat_add).to(self.device).contiguous()
            self._io_tables = (ay, ax, w_lat)
        ay, ax, w_lat = self._io_tables
        step, mb = divmod(self.loads, self.GAS)
        geom = DF.make_geom(self.ctx.grid, 1, self.replica_rank, sample0=self.c.dp * self.GAS + mb)
        return fused_io.IoPlan(geom, self.dcfg.sigma_data, (self.ecfg.seed << 32) + step, True, ay, ax, self._w_var,
                               w_lat, self.cfg.eps(self.cfg.data_dtype))

    # ------------------------------------------------------------------------------------------------ instructions
    def load(self, buffer_id):
        if not (self.is_first_stage() or self.is_last_stage()):
            return
        item = self.data_fn(self)                    # [1, H/wp_y, W/wp_x, C] blocks of this WP rank (+ interval, rit)
        cond_blk, tgt_blk = item[0], item[1]
        g = self.ctx.grid
        if self.fused_io and self.cfg.diffusion and self.noise_fn is None:
            # image blocks stay images: the kernels of the two end stages noise, embed, partition and score them
            x_img = tgt_blk.to(self.device, non_blocking=True).float().contiguous()
            if self.t_fn is not None:
                t = self.t_fn(self).to(self.device)
            else:
                t = TF.sample_noise_level(1, self.dcfg.sigma_min, self.dcfg.sigma_max, self.dcfg.sigma_data,
                                          generator=self.nl_rng, device=self.device, law=self.dcfg.noise_law)
            cs = torch.stack([torch.cos(t), torch.sin(t)], dim=1).float().contiguous()
            plan = self._io_plan()
            self.buf["x"][buffer_id], self.buf["z"][buffer_id], self.buf["t"][buffer_id] = (x_img, cs, plan), None, t
            if self.is_first_stage():
                c_img = cond_blk.to(self.device, non_blocking=True).float().contiguous()
                self.buf["inputs"][buffer_id] = (x_img, c_img, cs, plan)
            self.loads += 1
            return

        def to_tok(blk):
            B, hb, wb, C = blk.shape
            x = blk.to(self.device).view(B, g.nwy_loc, g.ws_y, g.nwx_loc, g.ws_x, C).permute(0, 1, 3, 2, 4, 5)
            return self._sp_slice(x.reshape(B * g.windows_per_rank * g.L, C).float())
        x = to_tok(tgt_blk)
        if not self.cfg.diffusion:
            # deterministic modes: the condition is the model input, the target the state to predict; the forecast
            # interval (rit) is the same on every rank that shares the sample (:286)
            t = None
            if self.cfg.rit:
                t = item[2].reshape(-1).float().to(self.device)
                rg = self.groups.get("replica")
                if rg is not None:
                    dist.broadcast(t, src=self.grid.replica_ranks(self.rank)[0], group=rg)
            self.buf["x"][buffer_id], self.buf["z"][buffer_id], self.buf["t"][buffer_id] = x, None, t
            self.loads += 1
            if self.is_first_stage():
                self.buf["inputs"][buffer_id] = to_tok(cond_blk)
            return
        if self.t_fn is not None:
            t = self.t_fn(self).to(self.device)
        else:
            t = TF.sample_noise_level(1, self.dcfg.sigma_min, self.dcfg.sigma_max, self.dcfg.sigma_data,
                                      generator=self.nl_rng, device=self.device, law=self.dcfg.noise_law)
        if self.noise_fn is not None:      # tests inject layout-independent noise
            z = to_tok(self.noise_fn(self)) * self.dcfg.sigma_data
        else:
            z = torch.randn(x.shape, generator=self.rng, device=self.device) * self.dcfg.sigma_data
        self.buf["x"][buffer_id], self.buf["z"][buffer_id], self.buf["t"][buffer_id] = x, z, t
        self.loads += 1
        if self.is_first_stage():
            c = to_tok(cond_blk)
            self.buf["inputs"][buffer_id] = TF.noise_inputs(x, c, z, t.repeat_interleave(x.shape[0]),
                                                            self.dcfg.sigma_data)

    def fwd(self, buffer_id):
        x = self.buf["inputs"][buffer_id]
        tgt = self.buf["x"][buffer_id]
        loss_io = tgt if (self.is_last_stage() and isinstance(tgt, tuple)) else None      # fused head + loss
        if self.is_first_stage():
            if isinstance(x, tuple):
                y, dt = self.module(None, None, self.buf["t"][buffer_id], self.ctx, images=x, loss_io=loss_io)
            else:
                y, dt = self.module(x, None, self.buf["t"][buffer_id], self.ctx, loss_io=loss_io)
        else:
            y, dt = self.module(x, self.buf["dt_in"][buffer_id], None, self.ctx, loss_io=loss_io)
        self.buf["outputs"][buffer_id], self.buf["dt_out"][buffer_id] = y, dt

    def bwd(self, buffer_id):
        out = self.buf["outputs"][buffer_id]
        if self.is_last_stage() and isinstance(self.buf["x"][buffer_id], tuple):
            self.loss_acc += out.detach().reshape(()).to(self.loss_acc.dtype)     # `out` is the loss itself
            out.backward()
        elif self.is_last_stage():
            x, z, t = self.buf["x"][buffer_id], self.buf["z"][buffer_id], self.buf["t"][buffer_id]
            if self.cfg.diffusion:
                tr = t.repeat_interleave(x.shape[0])
                sd = self.dcfg.sigma_data
                err = (sd * out - TF.v_target(x, z, tr)) ** 2 * self._w_var * self._w_lat
            else:
                err = (out - x) ** 2 * self._w_var * self._w_lat              # (:998)
            loss = err.sum(dim=-1).mean()
            self.loss_acc += loss.detach()
            loss.backward()
        elif self.dt_grad:
            # dt leaves this stage unchanged: on the first stage it is the embedding network's output, elsewhere the
            # received leaf, so the gradient from below is added to what this stage's own layers contribute
            torch.autograd.backward([out, self.buf["dt_out"][buffer_id]],
                                    [self.buf["grad_x"][buffer_id], self.buf["grad_dt"][buffer_id]])
        else:
            torch.autograd.backward(out, self.buf["grad_x"][buffer_id])
        for k in ("outputs", "x", "z", "grad_x", "grad_dt", "dt_out"):
            self.buf[k][buffer_id] = None

    # p2p ---------------------------------------------------------------------------------------------------------
    # One grouped transfer per instruction on the channel that :func:`schedule.p2p_op` names; x travels before dt and
    # the gradient of x before that of dt on both ends. Nothing here blocks the host on NCCL.
    def _wait_sends(self):
        self.links.wait_sends()

    def _act_buffers(self):
        B = 1
        x = torch.empty((self.tokens * B, self.cfg.dim), dtype=self.cfg.model_dtype, device=self.device)
        dt = torch.empty((B, self.cfg.dim), dtype=self.cfg.model_dtype, device=self.device)
        return x, dt

    def send(self, buffer_id):
        self.links.send("down_next", [self.buf["outputs"][buffer_id], self.buf["dt_out"][buffer_id]])

    def submit_recv(self, buffer_id):
        x, dt = self._act_buffers()
        self._pending[("act", buffer_id)] = (self.links.post_recv("down_prev", [x, dt]), x, dt)

    def process_recv(self, buffer_id):
        works, x, dt = self._pending.pop(("act", buffer_id))
        self.links.wait(works)
        self.buf["inputs"][buffer_id] = x.requires_grad_(True)   # leaf: its .grad is what goes back upstream
        # with one embedding network on the first stage (layerwise_t_emb off) dt is trainable upstream: a leaf too,
        # whose gradient (this stage's layers plus what the stages below send up) returns with that of x (:1052-1068)
        self.buf["dt_in"][buffer_id] = dt.requires_grad_(True) if self.dt_grad else dt

    def recv(self, buffer_id):
        self.submit_recv(buffer_id)
        self.process_recv(buffer_id)

    def send_grad(self, buffer_id):
        out = [self.buf["inputs"][buffer_id].grad]
        if self.dt_grad:
            g = self.buf["dt_in"][buffer_id].grad
            out.append(g if g is not None else torch.zeros_like(self.buf["dt_in"][buffer_id]))
        self.links.send("up_prev", out)
        self.buf["inputs"][buffer_id] = None
        self.buf["dt_in"][buffer_id] = None

    def submit_recv_grad(self, buffer_id):
        g = torch.empty((self.tokens, self.cfg.dim), dtype=self.cfg.model_dtype, device=self.device)
        bufs = [g]
        if self.dt_grad:
            bufs.append(torch.empty((1, self.cfg.dim), dtype=self.cfg.model_dtype, device=self.device))
        self._pending[("grad", buffer_id)] = (self.links.post_recv("up_next", bufs), bufs)

    def process_grad(self, buffer_id):
        works, bufs = self._pending.pop(("grad", buffer_id))
        self.links.wait(works)
        self.buf["grad_x"][buffer_id] = bufs[0]
        self.buf["grad_dt"][buffer_id] = bufs[1] if self.dt_grad else None

    def recv_grad(self, buffer_id):
        self.submit_recv_grad(buffer_id)
        self.process_grad(buffer_id)

    # reduce + step -------------------------------------------------------------------------------------------------
    def reduce_loss(self):
        if self.is_last_stage():
            lt = self.loss_acc / self.GAS
            g = self.groups.get("weight")
            if g is not None:
                dist.all_reduce(lt, group=g)
                lt = lt / dist.get_world_size(g)
            self.tot_loss = float(lt.item())
            self.loss_acc.zero_()

    def check_device(self):
        """Raise ``KernelError`` if a kernel recorded a device-side error (a bounded wait that ran out, a failed bounds
        check) since the last check; reads one word from the device."""
        if self.device.type == "cuda":
            from ..ops import lib as L
            L.check_status(sync=False)

    def reduce_grads(self):
        self._wait_sends()
        self.reduce_loss()
        self.check_device()       # before the gradients of an incomplete exchange reach the optimizer and the peers
        scale = 1.0 / (self.grid.DP * self.GAS)
        if not self.dcfg.grad_scale_parity:
            scale /= self.grid.WP_Y * self.grid.WP_X * self.grid.SP
        self._scale = scale
        if hasattr(self.opt, "reduce_scatter"):       # fused sharded optimizer: reduction and norm in one pass
            nsq = self.opt.reduce_scatter(scale)
            self._nsq = nsq
            if self.ocfg.grad_clip:
                self.stage_norm = float(nsq.item())
                if self.groups.get("pp") is not None:
                    dist.all_reduce(nsq, group=self.groups["pp"])
                self.total_norm = float(nsq.item()) ** 0.5
            return
        self.opt.reduce(self.groups.get("weight")) if hasattr(self.opt, "reduce") else self._allreduce_flat()
        if self.keep_grads:
            self.last_grads = {n: p.main_grad.clone() * scale for n, p in self.module.named_parameters()
                               if getattr(p, "main_grad", None) is not None}
        self._nsq = None
        if self.ocfg.grad_clip:
            nsq = self.opt.grad_norm_sq(scale)
            self.stage_norm = float(nsq.item())
            if self.groups.get("pp") is not None:
                dist.all_reduce(nsq, group=self.groups["pp"])
            self.total_norm = float(nsq.item()) ** 0.5
            self._nsq = nsq

    def _allreduce_flat(self):
        g = self.groups.get("weight")
        if g is None:
            return
        for b in self.opt.grad_buffers():
            dist.all_reduce(b, group=g)

    def step(self):
        if hasattr(self.opt, "reduce_scatter"):
            self.opt.apply(self.GAS * self.grid.DP, self._scale, self._nsq)
        else:
            self.opt.step(batch_img=self.GAS * self.grid.DP, grad_scale=self._scale, norm_sq=self._nsq)
        self.cur_it += 1

    # schedule execution --------------------------------------------------------------------------------------------
    def exec_schedule(self) -> dict[str, float]:
        timers: dict[str, float] = {}
        for cmds in self.schedule:
            for cmd in cmds:
                t0 = time.perf_counter()
                self._imap[type(cmd)](**cmd.kwargs)
                timers[cmd.name] = timers.get(cmd.name, 0.0) + time.perf_counter() - t0
        self._wait_sends()
        if self.device.type == "cuda":
            torch.cuda.synchronize()
            self.check_device()
        self.timers = timers
        e = self.ecfg
        if e.checkpoint_dir and not e.benchmark and self.cur_it % e.checkpoint_every == 0:
            self.save_checkpoint()
        return timers

    # checkpoints ---------------------------------------------------------------------------------------------------
    def save_checkpoint(self):
        """One file per logical stage, written by the head rank of each pipeline stage between two barriers (:1225-1234).
        With the distributed optimizer the state is sharded over the weight group: every rank takes part in the gathers
        and the head rank writes the same files (the reference cannot checkpoint in that mode, :1120-1122)."""
        dist.barrier() if dist.is_initialized() else None
        head = self.rank in self.grid.stage_heads()
        if head or self.ecfg.dist_optimizer or self.cfg.tp > 1:      # sharded state is gathered by all its holders
            numbered = self.cur_it % self.ecfg.checkpoint_keep_every == 0 and self.cur_it > 0
            save_stage_checkpoint(self.ecfg.checkpoint_dir, self.module, self.opt, it=self.cur_it if numbered else None,
                                  write=head)
        dist.barrier() if dist.is_initialized() else None

    def load_checkpoint(self) -> bool:
        ok = load_stage_checkpoint(self.ecfg.checkpoint_dir, self.module, self.opt, self.device)
        if ok:
            # continue the noise streams where a run of this length would be (:1155-1156)
            self.rng.manual_seed(self.cur_nimg + self._noise_seed)
            self.nl_rng.manual_seed(self.cur_nimg + self.ecfg.seed + self.c.dp)
        if dist.is_initialized():
            dist.barrier()
        return ok

    # warm-up straggler probe -----------------------------------------------------------------------------------------
    def warmup(self, iters: int = 3, threshold: float = 1.08) -> dict:
        """Times a few forward/backward passes of this stage on random input and flags ranks more than 8 % slower
        than the mean of their weight group (:1492-1533). Returns {"time", "mean", "slow"}."""
        if self.is_first_stage() and not self.module.layer_ids:
            return {"time": 0.0, "mean": 0.0, "slow": False}
        x = torch.randn((self.tokens, self.cfg.dim), device=self.device).to(self.cfg.model_dtype)
        dt = torch.zeros((1, self.cfg.dim), device=self.device, dtype=self.cfg.model_dtype)
        layers_only = PipelineStageView(self.module)

        def once():
            xin = x.clone().requires_grad_(True)
            y = layers_only(xin, dt, self.ctx)
            y.float().pow(2).mean().backward()
        for _ in range(iters):
            once()
        if self.device.type == "cuda":
            torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(iters):
            once()
        if self.device.type == "cuda":
            torch.cuda.synchronize()
        took = time.perf_counter() - t0
        self.opt.zero_grad()
        mean = took
        g = self.groups.get("weight")
        if g is not None:
            tt = torch.tensor([took], device=self.device, dtype=torch.float64)
            dist.all_reduce(tt, group=g)
            mean = float(tt.item()) / dist.get_world_size(g)
        slow = took > mean * threshold
        if slow:
            print(f"ALERT, slow warmup on rank {self.rank} ({100 * took / mean:.1f}%), time {took:.3f}, avg {mean:.3f}",
                  flush=True)
        return {"time": took, "mean": mean, "slow": slow}


class PipelineStageView:
    """Runs only the Swin layers of a stage (warm-up probe)."""

    def __init__(self, stage: PipelineStage):
        self.stage = stage

    def __call__(self, x, dt, ctx):
        st = self.stage
        cur = st.entry_shift()
        for i in st.layer_ids:
            nxt = st.cfg.layer_shift(i)
            x = st.layers[str(i)](x, dt, ctx, regroup=(cur, nxt))
            cur = nxt
        return x
