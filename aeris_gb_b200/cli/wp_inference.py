"""WP-only autoregressive ensemble inference.

    torchrun --nproc-per-node 8 -m aeris_gb_b200.cli.wp_inference --checkpoint DIR --WP-Y 2 --WP-X 4 --members 4
    torchrun --nproc-per-node 8 -m aeris_gb_b200.cli.wp_inference --checkpoint DIR --member-parallel --members 8

Reference: src/aeris_wp_inference/inference.py (argparse CLI :24-41, rollout :43-198, mesh [DP, SP=WP] :215-231,
checkpoint conversion :281, strided initial conditions :302-314). Two layouts: every member window-parallel over all
GPUs (the reference's), or one member per GPU (``--member-parallel``: no halo traffic at all, members are independent
until the metrics). The state stays on the device for the whole rollout. ``--data FILE`` (``--data-root`` = folder of
the statistics files) reads initial conditions every ``--stride-ic`` samples, split over the data-parallel replicas,
with forcings and verification fields from the file, dataset statistics for the (un)standardisation and, with
``--out``, the rollout of every window-parallel tile written per forecast step. Without ``--data`` synthetic N(0,1)
initial states and forcings are used, and with ``--random-init`` random weights (benchmarking without a checkpoint).
"""
from __future__ import annotations

import argparse
import json
import os
import time

import numpy as np
import torch
import torch.distributed as dist

from ..data.sharding import gather_blocks, shard_block
from ..diffusion.rollout import DeviceForecaster, Forecaster, SamplerConfig
from ..diffusion import trigflow as TF
from ..engine.checkpoint import convert_inference_checkpoint
from ..eval.metrics import EnsembleMetrics
from ..models import layout as LY
from ..models.aeris import AerisModel, StreamContext
from ..parallel.symm import HaloExchange
from ..utils import config as C
from ..utils.dist_setup import setup, teardown
from ..utils.io import print0


def parse(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--checkpoint", default=None)
    ap.add_argument("--experiment", default="b200_wp_inference")
    ap.add_argument("--WP-Y", type=int, default=1)
    ap.add_argument("--WP-X", type=int, default=1)
    ap.add_argument("--member-parallel", action="store_true")
    ap.add_argument("--members", type=int, default=1)
    # the second spelling of an option is the reference's (aeris_wp_inference/inference.py:24-41)
    ap.add_argument("--rollout-steps", "--steps", dest="rollout_steps", type=int, default=None)
    ap.add_argument("--sampler-steps", "--diffusion-steps", dest="sampler_steps", type=int, default=None)
    ap.add_argument("--stride-ic", "--stride", dest="stride_ic", type=int, default=1)
    ap.add_argument("--start-sample", type=int, default=-1, help="first initial condition of the file (-1: the first)")
    ap.add_argument("--end-sample", type=int, default=-1, help="last initial condition (-1: as many as fit)")
    ap.add_argument("--extra-name", default="", help="text in front of the checkpoint file names, e.g. it_5000_")
    ap.add_argument("--sequence-parallel", type=int, default=None,
                    help="accepted: the reference wants WP_Y x WP_X here; the window-parallel grid alone decides")
    ap.add_argument("--S_churn", "--S-churn", dest="S_churn", type=float, default=0.0)
    ap.add_argument("--S_min", "--S-min", dest="S_min", type=float, default=0.0)
    ap.add_argument("--S_max", "--S-max", dest="S_max", type=float, default=float("inf"))
    ap.add_argument("--S_noise", "--S-noise", dest="S_noise", type=float, default=1.0)
    ap.add_argument("--sigma_max", "--sigma-max", dest="sigma_max", type=float, default=-1.0,
                    help="largest noise level of the sampler (-1: the model's)")
    ap.add_argument("--sigma_min", "--sigma-min", dest="sigma_min", type=float, default=-1.0)
    ap.add_argument("--data", default=None, help="monolithic test file [T, 73, 721, 1440]")
    ap.add_argument("--data-root", default=None)
    ap.add_argument("--out", default=None)
    ap.add_argument("--random-init", action="store_true")
    ap.add_argument("--no-ema", action="store_true")
    ap.add_argument("--euler", action="store_true")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--debug", action="store_true")
    ap.add_argument("--local-eval", action="store_true",
                    help="print the running first-channel (2 m temperature) scores after every rollout step")
    ap.add_argument("overrides", nargs="*")
    return ap.parse_args(argv)


def main(argv=None):
    a = parse(argv)
    rank, world, device = setup()
    if a.checkpoint and os.path.exists(os.path.join(a.checkpoint, ".hydra", "config.yaml")):
        cfg = C.load_run_config(a.checkpoint)
    else:
        cfg = C.compose("train", [f"experiment={a.experiment}"] + list(a.overrides))
    wp = (1, 1) if a.member_parallel else (a.WP_Y, a.WP_X)
    cfg.model.WP_Y, cfg.model.WP_X = wp
    mcfg = C.model_config(cfg)
    mcfg.tp = 1       # inference holds whole MLP weights; checkpoints store full tensors whatever model.TP trained them
    if device.type == "cpu":
        mcfg.model_dtype = torch.float32
    n_wp = wp[0] * wp[1]
    assert world % n_wp == 0
    dp = world // n_wp
    dp_rank, wp_rank = rank // n_wp, rank % n_wp
    wp_group = None
    if n_wp > 1:
        for d in range(dp):
            g = dist.new_group(list(range(d * n_wp, (d + 1) * n_wp)))
            if d == dp_rank:
                wp_group = g
    torch.manual_seed(a.seed)
    model = AerisModel(mcfg).to(device).eval()
    if a.checkpoint and not a.random_init:
        convert_inference_checkpoint(a.checkpoint, mcfg.n_layers + 2, model, use_ema=not a.no_ema, strict=False,
                                     prefix=a.extra_name)
    halo = HaloExchange(wp_group, device) if (n_wp > 1 and device.type == "cuda") else None
    grid = mcfg.grid()
    H, W = mcfg.img
    hb, wb = H // wp[0], W // wp[1]
    C_out = mcfg.out_channels
    C_f = mcfg.in_channels - 2 * C_out
    steps = a.rollout_steps or int(cfg.model.get("rollout_steps", 4))
    sampler = SamplerConfig(n_steps=a.sampler_steps or int(cfg.model.get("sampler_steps", 20)),
                            sigma_min=cfg.model.sigma_min if a.sigma_min < 0 else a.sigma_min,
                            sigma_max=cfg.model.sigma_max if a.sigma_max < 0 else a.sigma_max,
                            sigma_data=cfg.model.sigma_data, heun=not a.euler, s_churn=a.S_churn, s_min=a.S_min,
                            s_max=a.S_max, s_noise=a.S_noise)
    # members handled by this rank: all of them when window-parallel, a strided subset when member-parallel
    my_members = list(range(dp_rank, a.members, dp)) if a.member_parallel else list(range(a.members))
    M = len(my_members)
    ctx = StreamContext(mcfg, max(M, 1), wp_rank, halo.peer_fn if halo else None, wp_group=wp_group)

    def denoise(model_in, t):
        B = model_in.shape[0]
        tok = model_in.reshape(B * hb * wb, -1)
        g = grid
        tok = model_in.view(B, g.nwy_loc, g.ws_y, g.nwx_loc, g.ws_x, -1).permute(0, 1, 3, 2, 4, 5).reshape(B * g.tokens_per_rank, -1)
        out = model.forward_tokens(tok, t, ctx)
        out = out.view(B, g.nwy_loc, g.nwx_loc, g.ws_y, g.ws_x, -1).permute(0, 1, 3, 2, 4, 5)
        return out.reshape(B, hb, wb, -1).float()

    wp_yx = (wp_rank // wp[1], wp_rank % wp[1])
    data = None
    if a.data:
        from ..data.inference_data import InferenceData, RolloutWriter, strided_indices
        data = InferenceData(a.data, a.data_root, (H, W), wp, wp_yx, interval=int(cfg.model.get("interval", 6)),
                             rollout_steps=steps, out_channels=C_out,
                             channels=73 if C_f > 0 else 69)
        stats = data.stats(device)
        # window-parallel: the replicas share the initial conditions out; member-parallel: every rank sees all of them
        all_ic, my_ic = strided_indices(data.ds.ds.shape[0], steps, data.dt, a.stride_ic,
                                        0 if a.member_parallel else dp_rank, 1 if a.member_parallel else dp,
                                        start=max(a.start_sample, 0), end=None if a.end_sample < 0 else a.end_sample)
    else:
        stats = {k: torch.zeros(C_out, device=device) if "mean" in k else torch.ones(C_out, device=device)
                 for k in ("x_mean", "x_std", "t_mean", "t_std")}
        all_ic = my_ic = [0]
    gen = torch.Generator(device=device).manual_seed(a.seed * 1000 + rank)
    if device.type == "cuda":     # sampler, (un)standardisation, embedding and head on the CUDA kernels
        fc = DeviceForecaster(model, ctx, stats, sampler, C_out, seed=a.seed,
                              member0=(dp_rank * ((a.members + dp - 1) // dp) if a.member_parallel else 0))
    else:
        fc = Forecaster(denoise, stats, sampler, C_out)
    w_lat = TF.latitude_weights(H, float(cfg.model.get("w_lat_add", 0.0))).to(device)
    w_lat_blk = w_lat.view(wp[0], hb)[wp_rank // wp[1]]
    metrics = EnsembleMetrics(steps, C_out, H * W, device, group=wp_group)
    g0 = torch.Generator().manual_seed(a.seed)
    state_full = torch.randn(H, W, C_out, generator=g0)
    truth_full = [torch.randn(H, W, C_out, generator=g0) for _ in range(steps)] if a.debug else None
    syn_forcing = torch.randn(max(M, 1), hb, wb, C_f, generator=gen, device=device) if C_f > 0 else None
    writer = None
    if a.out and data is not None and M > 0:
        stem = f"rollout-{len(all_ic)}i-{steps}s-{a.members}m" + (f"_dp{dp_rank}" if dp > 1 else "")
        writer = RolloutWriter(a.out, stem, wp_yx, len(my_ic), steps, M, C_out, hb, wb)
    times = []
    cur = {}

    def on_step(k, x):
        if device.type == "cuda":
            torch.cuda.synchronize()
            from ..ops import lib as L
            L.check_status(sync=False)         # a bounded device wait that ran out ends the rollout here
        times.append(time.perf_counter())
        if writer is not None:
            writer.put(cur["ic"], k + 1, x)
        if a.member_parallel and world > 1:
            allm = [torch.empty_like(x) for _ in range(world)]
            dist.all_gather(allm, x)
            mem = torch.cat(allm).permute(0, 3, 1, 2)
        else:
            mem = x.permute(0, 3, 1, 2)
        metrics.update(k, mem, cur["truth"](k), w_lat_blk)
        if a.local_eval:
            print0(metrics.running_line(k, 0, int(cfg.model.get("interval", 6))))

    t_start = time.perf_counter()
    times.append(t_start)
    for n, idx in enumerate(my_ic):
        if data is not None:
            smp = data.sample(idx)
            state = smp["state"].to(device).unsqueeze(0).repeat(max(M, 1), 1, 1, 1)
            f_all = smp["forcing"].to(device) if smp["forcing"] is not None else None
            forcings = (lambda k: f_all[k].unsqueeze(0).expand(max(M, 1), -1, -1, -1)) if f_all is not None else None
            truth = smp["truth"].to(device)
            cur.update(ic=n, truth=lambda k: truth[k].permute(2, 0, 1))
        else:
            state = shard_block(state_full.unsqueeze(0), wp, wp_yx).to(device).repeat(max(M, 1), 1, 1, 1)
            forcings = (lambda k: syn_forcing) if syn_forcing is not None else None
            label = lambda k: shard_block((truth_full[k] if truth_full is not None else state_full).unsqueeze(0), wp,
                                          wp_yx)[0].to(device).permute(2, 0, 1)
            cur.update(ic=n, truth=label)
        if writer is not None:
            writer.put(n, 0, state)
        if M > 0:
            fc.rollout(state, forcings, steps, generator=gen, on_step=on_step)
        metrics.end_initial_condition()
    if dp > 1 and not a.member_parallel:        # scores of the replicas' initial conditions in one packed reduction
        packed = torch.cat([metrics.err.reshape(-1), torch.tensor([float(metrics.count)], device=device,
                                                                  dtype=torch.float64)])
        dist.all_reduce(packed)
        metrics.err = packed[:-1].view_as(metrics.err) / n_wp       # every WP rank of a replica holds the same sums
        metrics.count = int(round(packed[-1].item() / n_wp))
    agg, scores = metrics.finalize()
    if writer is not None:
        writer.close()
    if mcfg.out_channels in (69, 70):   # the named channel sets: scores of the nine headline variables
        from ..data.era5 import variable_names
        print0("RMSE first member, RMSE ensemble mean, CRPS, spread/skill\n"
               + metrics.headline_table(variable_names(73)[:mcfg.out_channels], interval=int(cfg.model.get("interval", 6))))
    per_step = float(np.mean(np.diff(times))) if len(times) > 1 else float("nan")
    if a.out and rank == 0:
        os.makedirs(a.out, exist_ok=True)
        np.save(os.path.join(a.out, "rollout_err_aggregate.npy"), agg)
        np.save(os.path.join(a.out, "rollout_err.npy"), scores)
    print0(json.dumps({"entry": "wp_inference", "world": world, "wp": list(wp), "member_parallel": a.member_parallel,
                       "members": a.members, "rollout_steps": steps, "sampler_steps": sampler.n_steps,
                       "model_evals_per_step": fc.model_evals_per_forecast_step(), "s_per_forecast_step": per_step,
                       "rmse_t2m_first_step": float(scores[0, 0, 0])}))
    teardown()


if __name__ == "__main__":
    main()
