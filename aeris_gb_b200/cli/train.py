"""Training entry point.

    python -m aeris_gb_b200.cli.train experiment=b200_1p3b_wp8 data.synthetic=true trainer.benchmark_steps=20
    torchrun --nproc-per-node 8 -m aeris_gb_b200.cli.train experiment=b200_1p3b_wp8

Same flow as the reference's Hydra main (src/aeris/train.py:66-358): bootstrap, seeds, dataset, channel wiring, engine,
optimizer policy, warm-up probe, checkpoint load, data loader, main loop with TFLOP/s per GPU, periodic checkpoints.
Overrides are ``key=value`` (dotted) like Hydra's. With ``model.PP = 1`` the single-node fused engine (:class:`Trainer`:
WP x SP x DP, every logical stage on every GPU) runs the step; otherwise the pipeline engine (:class:`ParallelEngine`).
"""
from __future__ import annotations

import os
import sys
import time

import torch
import torch.distributed as dist

from ..data.samplers import InfiniteSampler
from ..data.synthetic import SyntheticERA5
from ..engine.checkpoint import load_stage_checkpoint, save_stage_checkpoint
from ..engine.optim import FlatOptimizer
from ..engine.pipeline import EngineConfig, ParallelEngine
from ..engine.trainer import Trainer
from ..parallel.topology import ProcessGrid
from ..utils import config as C
from ..utils.dist_setup import setup, teardown
from ..utils.fault import FaultInjector, Heartbeat, StepWatchdog, check_finite
from ..utils.io import log0
from ..utils.timers import memory_report, tflops_per_gpu, wandb_payload


def build_dataset(cfg, mcfg, wp_rank, channels):
    rti = mcfg.rit and not mcfg.diffusion
    if cfg.data.get("synthetic", False) or not cfg.data.get("root"):
        cond = channels["condition"] if mcfg.diffusion else channels["model_in"]
        return SyntheticERA5(img=mcfg.img, cond_channels=cond, target_channels=channels["label"],
                             wp=mcfg.wp, wp_rank=wp_rank, seed=int(cfg.seed), intervals=(6, 12, 24) if rti else None)
    if rti:
        from ..data.era5 import ERA5NRMRTIDataset
        ds = ERA5NRMRTIDataset(cfg.data.dataset.root, cfg.data.root, interval=int(cfg.model.interval),
                               channels=channels["dataset"], seed=int(cfg.seed))
        ds.open_file(wp_rank[0], wp_rank[1], benchmark=bool(cfg.model.get("benchmark", False)),
                     data_shape=(30, channels["dataset"], mcfg.img[0] // mcfg.wp[0], mcfg.img[1] // mcfg.wp[1]))
        return _ChannelsLast(ds)
    from ..data.era5 import ERA5NRMDataset
    ds = ERA5NRMDataset(cfg.data.dataset.root, cfg.data.root, interval=int(cfg.model.interval),
                        channels=channels["dataset"])
    ds.open_file(wp_rank[0], wp_rank[1], load_x=True, load_t=True, benchmark=bool(cfg.model.get("benchmark", False)))
    return _ChannelsLast(ds)


class _ChannelsLast(torch.utils.data.Dataset):
    """ERA5 items are [C, H, W]; the engines take [H, W, C] blocks."""

    def __init__(self, ds):
        self.ds = ds

    def __len__(self):
        return len(self.ds)

    def __getitem__(self, i):
        x, t, *rest = self.ds[i]
        return (x.permute(1, 2, 0).contiguous(), t.permute(1, 2, 0).contiguous(), *rest)


def _module_norm(module) -> float:
    """L2 norm of all parameters of a module (src/aeris/train.py:300-307)."""
    return float(torch.sqrt(sum(p.detach().float().pow(2).sum() for p in module.parameters())))


def stage_metrics(layers: dict, stage_norm: float | None, pp_rank: int, n_stages: int, timers: dict | None) -> dict:
    """What one rank per pipeline stage logs (train.py:322-340): the stage's gradient norm, the norms of the two
    modulation matrices of the first block of the first and last Swin stage, per-instruction timers."""
    out = {}
    if stage_norm is not None:
        out[f"train/stage_norm/stage_norm_{pp_rank}"] = stage_norm
    for stage, layer in layers.items():
        if stage in (1, n_stages - 2) and len(layer.modulelist[0][4].modulation) == 3:
            mod = layer.modulelist[0][4].modulation
            out[f"train/weight_norm/stage_{stage}/0_modulation_0"] = _module_norm(mod[0])
            out[f"train/weight_norm/stage_{stage}/0_modulation_2"] = _module_norm(mod[2])
    for k, v in (timers or {}).items():
        out[f"train/pp_timers/{k}/rank_{pp_rank}"] = v
    return out


def main(argv=None):
    argv = list(sys.argv[1:] if argv is None else argv)
    cfg = C.compose("train", argv)
    rank, world, device = setup()
    torch.manual_seed(int(cfg.seed) + rank)
    mcfg, ocfg, dcfg = C.model_config(cfg), C.optim_config(cfg), C.diffusion_config(cfg)
    if str(cfg.model.get("dtype", "bfloat16")) == "float32" or device.type == "cpu":
        mcfg.model_dtype = torch.float32
    channels = C.channel_counts(cfg)
    PP, SP = int(cfg.model.get("PP", 1)), int(cfg.model.get("SP", 1))
    gas = int(cfg.data.gas)
    grid = ProcessGrid(world, PP=PP, SP=SP, WP_Y=mcfg.wp[0], WP_X=mcfg.wp[1])
    log0(grid.describe())
    c = grid.coords(rank)
    ckpt_dir = cfg.model.get("checkpoint_dir")
    if rank == 0 and ckpt_dir:
        C.save_run_config(cfg, ckpt_dir)
    ds = build_dataset(cfg, mcfg, (c.wp_y, c.wp_x), channels)

    def make_loader(cur_nimg: int):
        # built after the checkpoint is loaded: a resumed run continues with another sample order (train.py:247)
        sampler = InfiniteSampler(ds, rank=c.dp, num_replicas=grid.DP, seed=int(cfg.seed) + cur_nimg)
        workers = 0 if isinstance(ds, SyntheticERA5) else int(cfg.data.data_workers)
        return iter(torch.utils.data.DataLoader(ds, sampler=sampler, batch_size=1, num_workers=workers,
                                                pin_memory=device.type == "cuda"))
    steps = int(cfg.trainer.get("benchmark_steps", -1))
    total_steps = steps if steps > 0 else max(1, int(cfg.trainer.total_kimg * 1000) // (gas * grid.DP))
    watchdog = StepWatchdog()
    # liveness between steps: every rank beats into the rendezvous store; a rank that stopped is reported before the
    # next step launches anything that would wait for it. AERIS_FAULT injects host-side failures (utils/fault.py).
    injector = FaultInjector()
    heart = None
    if world > 1 and dist.is_initialized():
        store = getattr(dist.distributed_c10d, "_get_default_store", lambda: None)()
        if store is not None:
            heart = Heartbeat(store, rank, world, timeout_s=float(cfg.trainer.get("heartbeat_timeout_s", 600.0)))

    def between_steps(it: int):
        injector.maybe_raise(rank, it)
        if heart is not None:
            if not injector.silences(rank, it):
                heart.beat()
            heart.check()
    wandb = None
    if os.environ.get("WANDB_MODE", "disabled") != "disabled" and (rank == 0 or rank in grid.stage_heads()):
        try:
            import wandb as _w
            wandb = _w
            wandb.init(project="aeris", config=cfg.to_dict(), group=str(cfg.get("experiment_name", "aeris")),
                       name=f"rank{rank}")
        except Exception:
            wandb = None
    n_logical = mcfg.n_layers + 2

    if PP == 1 and (SP == 1 or device.type == "cuda"):
        # one process group per sample (WP x SP ranks, ordered wp_y, wp_x, sp), its SP sub-groups, and the weight group
        tp_on = mcfg.tp > 1             # model.TP: the MLP weights split over the SP group (or the WP group)
        kinds = ("replica", "sp", "weight") + (("tp", "tp_ortho") if tp_on else ())
        groups = grid.build_groups(rank, kinds=kinds) if world > 1 else {}
        mcfg.sp = SP
        if tp_on:
            tp_ranks = grid.tp_ranks(rank)
            if mcfg.tp != len(tp_ranks):
                raise SystemExit(f"model.TP = {mcfg.tp} must equal the size of the tensor-parallel group "
                                 f"({len(tp_ranks)}: SP when SP > 1, else WP_Y x WP_X)")
            mcfg.tp_rank = tp_ranks.index(rank)
        trainer = Trainer(mcfg, ocfg, dcfg, device, seed=int(cfg.seed), wp_group=groups.get("replica"),
                          dp_size=grid.DP, dp_rank=c.dp, weight_group=groups.get("weight"),
                          sp_group=groups.get("sp"), tp_group=groups.get("tp"), tp_ortho_group=groups.get("tp_ortho"))
        trainer.timers.enabled = bool(cfg.trainer.get("report_timings", False))
        if cfg.model.get("load") and ckpt_dir:
            if load_stage_checkpoint(ckpt_dir, trainer.model, trainer.opt, device):
                trainer.resume(trainer.opt.cur_nimg, gas)
                log0(f"loaded a checkpoint from {ckpt_dir} at {trainer.opt.cur_nimg} images")
        loader = make_loader(trainer.opt.cur_nimg)
        start = trainer.opt.cur_nimg // (gas * grid.DP)
        # trainer.profile_steps=[first,last): torch.profiler Chrome trace of those iterations, one file per rank
        from ..utils.timers import StepProfiler
        ps = cfg.trainer.get("profile_steps")
        prof = StepProfiler(tuple(int(v) for v in ps) if ps else None,
                            os.path.join(ckpt_dir or ".", "traces"), rank)
        for it in range(start, total_steps):
            between_steps(it)
            prof.before_step(it)
            batch = [next(loader) for _ in range(gas)]
            cond = torch.cat([b[0] for b in batch]).pin_memory() if device.type == "cuda" else torch.cat([b[0] for b in batch])
            tgt = torch.cat([b[1] for b in batch]).pin_memory() if device.type == "cuda" else torch.cat([b[1] for b in batch])
            tgt = injector.poison(tgt, rank, it)
            interval = torch.cat([b[2] for b in batch]).reshape(-1) if len(batch[0]) > 2 else None
            t0 = time.perf_counter()
            loss = trainer.train_step(tgt, cond, interval=interval)
            dt = time.perf_counter() - t0
            trace = prof.after_step(it)
            if trace:
                log0(f"profiler trace written to {trace}")
            check_finite("loss", loss)
            tf = tflops_per_gpu(mcfg.flops_per_sample(), gas * grid.DP, dt, world)
            slow = watchdog.observe(dt)
            log0(f"it {it} loss {loss:.5f} |g| {trainer.grad_norm():.4f} {dt:.3f} s/it {tf:.1f} TFLOP/s/GPU"
                 + (" SLOW STEP" if slow else "")
                 + ((" " + memory_report(device)) if cfg.model.get("benchmark") else ""))
            phase = trainer.timers.resolve() if trainer.timers.enabled else None
            if phase:
                log0("   device ms: " + str({k: round(v, 1) for k, v in phase.items()}))
            if wandb and rank == 0:
                payload = wandb_payload(it, trainer.opt.cur_nimg, tf, dt, loss, trainer.grad_norm(), trainer.opt.last_lr)
                payload.update(stage_metrics({i + 1: l for i, l in enumerate(trainer.model.layers)},
                                             trainer.grad_norm() ** 2, 0, n_logical, phase))
                wandb.log(payload)
            every = int(cfg.trainer.get("checkpoint_every", 100))
            if ckpt_dir and not cfg.model.get("benchmark") and (it + 1) % every == 0:
                # the sharded optimizer gathers its state over the group, so every rank calls; one rank writes, and
                # nobody runs ahead into the next step's device barriers while it does
                if rank == 0 or not isinstance(trainer.opt, FlatOptimizer):
                    save_stage_checkpoint(ckpt_dir, trainer.model, trainer.opt,
                                          it=(it + 1) if (it + 1) % 1000 == 0 else None, write=(rank == 0))
                if world > 1:
                    dist.barrier()
    else:
        ecfg = EngineConfig(gas=gas, overlap_p2p=bool(cfg.model.get("overlap_p2p_comms", False)),
                            dist_optimizer=bool(cfg.model.get("dist_optimizer", False)),
                            rs_grads=bool(cfg.model.get("rs_grads", True)), checkpoint_dir=ckpt_dir,
                            benchmark=bool(cfg.model.get("benchmark", False)), seed=int(cfg.seed),
                            init_policy={k: cfg.model.get(k) for k in
                                         ("init_scale_test14", "init_scale_test15", "time_emb_init", "head_init_std",
                                          "token_emb_init_std", "modulation_0_init", "modulation_2_init")
                                         if cfg.model.get(k) is not None})
        holder = {}

        def data_fn(_eng):
            return next(holder["loader"])        # (condition, target[, interval])
        mcfg.sp = SP
        eng = ParallelEngine(mcfg, ocfg, dcfg, ecfg, grid, rank, device, data_fn=data_fn)
        eng.warmup()
        if cfg.model.get("load"):
            eng.load_checkpoint()
        holder["loader"] = make_loader(eng.cur_nimg)
        for it in range(eng.cur_nimg // (gas * grid.DP), total_steps):
            between_steps(it)
            t0 = time.perf_counter()
            timers = eng.exec_schedule()
            dt = time.perf_counter() - t0
            tf = tflops_per_gpu(mcfg.flops_per_sample(), gas * grid.DP, dt, world)
            if eng.is_last_stage() and c.dp == 0 and c.wp_y == 0 and c.wp_x == 0 and c.sp == 0:
                check_finite("loss", eng.tot_loss)
                print(f"it {it} loss {eng.tot_loss:.5f} |g| {eng.total_norm:.4f} {dt:.3f} s/it {tf:.1f} TFLOP/s/GPU"
                      + ((" " + memory_report(device)) if cfg.model.get("benchmark") else ""), flush=True)
            report = bool(cfg.trainer.get("report_timings"))
            if report and rank in grid.stage_heads():
                print(c.pp, "times:", {k: round(v, 4) for k, v in timers.items()}, flush=True)
            if wandb:
                payload = {}
                if rank == 0:
                    payload.update(wandb_payload(it, eng.cur_nimg, tf, dt))
                if rank in grid.stage_heads():
                    layers = {int(i) + 1: l for i, l in eng.module.layers.items()}
                    payload.update(stage_metrics(layers, eng.stage_norm, c.pp, n_logical, timers if report else None))
                    if eng.is_last_stage():
                        payload.update({"train/loss": eng.tot_loss, "train/total_norm": eng.total_norm,
                                        "lr": eng.opt.last_lr})
                wandb.log(payload, step=it)
    if heart is not None:
        heart.mark_leaving()
    if cfg.trainer.get("sleep_after_done"):     # keeps the job's allocation alive after the last step (train.py:350-351)
        time.sleep(100000)
    teardown()


if __name__ == "__main__":
    main()
