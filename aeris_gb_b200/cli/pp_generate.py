"""Pipeline-parallel ensemble inference with on-the-fly scores.

    torchrun --nproc-per-node 8 -m aeris_gb_b200.cli.pp_generate --checkpoint DIR --PP 2 --WP-Y 1 --WP-X 2 --members 4

Reference: src/aeris/pp_generate.py (CLI :28-53, rollout :62-526, sampler :113-119/:298-322, metrics :346-472, output
files :93-99/:486-496). The sampler runs on the first pipeline stage and pushes every network evaluation through the
pipeline with the ensemble members as micro-batches; the autoregressive state stays on the device. ``--data`` reads
strided initial conditions (split over the data-parallel replicas, :611-637), forcings and verification fields from a
test file and (un)standardises with its statistics; ``--out`` then also writes every tile's rollout. ``--S-churn``
adds the stochastic churn step (:228-241). Without ``--checkpoint`` random weights, without ``--data`` synthetic N(0,1)
fields are used.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import time

import numpy as np
import torch
import torch.distributed as dist

from ..diffusion import trigflow as TF
from ..engine.inference import InferenceEngine
from ..engine.optim import OptimConfig
from ..engine.pipeline import EngineConfig
from ..engine.trainer import DiffusionConfig
from ..eval.metrics import EnsembleMetrics
from ..models import layout as LY
from ..parallel.topology import ProcessGrid
from ..utils import config as C
from ..utils.dist_setup import setup, teardown
from ..utils.io import print0


def parse(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--checkpoint", default=None)
    ap.add_argument("--experiment", default="b200_wp_inference")
    ap.add_argument("--PP", type=int, default=1)
    ap.add_argument("--WP-Y", type=int, default=1)
    ap.add_argument("--WP-X", type=int, default=1)
    ap.add_argument("--members", type=int, default=2)
    # the second spelling of an option is the reference's (pp_generate.py:28-53)
    ap.add_argument("--rollout-steps", "--steps", dest="rollout_steps", type=int, default=2)
    ap.add_argument("--sampler-steps", "--diffusion-steps", dest="sampler_steps", type=int, default=20)
    ap.add_argument("--S-churn", "--S_churn", dest="S_churn", type=float, default=0.0)
    ap.add_argument("--S-min", "--S_min", dest="S_min", type=float, default=0.0)
    ap.add_argument("--S-max", "--S_max", dest="S_max", type=float, default=float("inf"))
    ap.add_argument("--S-noise", "--S_noise", dest="S_noise", type=float, default=1.0)
    ap.add_argument("--sigma_max", "--sigma-max", dest="sigma_max", type=float, default=-1.0,
                    help="largest noise level of the sampler (-1: the model's)")
    ap.add_argument("--sigma_min", "--sigma-min", dest="sigma_min", type=float, default=-1.0)
    ap.add_argument("--start-sample", type=int, default=-1, help="first initial condition of the file (-1: the first)")
    ap.add_argument("--end-sample", type=int, default=-1, help="last initial condition (-1: as many as fit)")
    ap.add_argument("--extra-name", default="", help="text in front of the checkpoint file names, e.g. it_5000_")
    ap.add_argument("--extra-outname", default="", help="text appended to the name of the rollout files")
    ap.add_argument("--local-eval", action="store_true",
                    help="print the running first-channel (2 m temperature) scores after every rollout step")
    ap.add_argument("--clamp-sst", action="store_true",
                    help="accepted: land points of the sea-surface temperature are always filled before standardising")
    ap.add_argument("--euler", action="store_true")
    ap.add_argument("--load-ema", "--use-ema", dest="load_ema", action="store_true", help="take the EMA weights of the checkpoint (default: the model weights)")
    ap.add_argument("--data", default=None, help="monolithic test file [T, 73, 721, 1440]")
    ap.add_argument("--data-root", default=None, help="folder with the normalize_*.npz statistics")
    ap.add_argument("--stride-ic", "--stride", dest="stride_ic", type=int, default=1)
    ap.add_argument("--out", default=None)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("overrides", nargs="*")
    return ap.parse_args(argv)


def churn_rotation(s_cur: float, n_steps: int, S_churn: float, S_min: float, S_max: float) -> tuple[float, float]:
    """(raised noise level s, rotation angle s_l) of the churn step, form 2 (pp_generate.py:228-241):
    gamma = min(S_churn / N, sqrt 2 - 1) inside [S_min, S_max] (in units of tan s), s = atan((1 + gamma) tan s_cur),
    s_l = atan(tan s - tan s_cur); the state is rotated toward fresh noise by s_l."""
    gamma = min(S_churn / n_steps, math.sqrt(2) - 1) if (S_churn > 0 and S_min <= math.tan(s_cur) <= S_max) else 0.0
    s = math.atan((1 + gamma) * math.tan(s_cur))
    return s, math.atan(math.tan(s) - math.tan(s_cur))


def main(argv=None):
    a = parse(argv)
    rank, world, device = setup()
    if a.checkpoint and os.path.exists(os.path.join(a.checkpoint, ".hydra", "config.yaml")):
        cfg = C.load_run_config(a.checkpoint)
        for ov in a.overrides:
            k, _, v = ov.partition("=")
            cfg.set_path(k.lstrip("+"), C._parse_value(v))
    else:
        cfg = C.compose("train", [f"experiment={a.experiment}"] + list(a.overrides))
    cfg.model.WP_Y, cfg.model.WP_X = a.WP_Y, a.WP_X
    mcfg = C.model_config(cfg)
    mcfg.tp = 1       # inference holds whole MLP weights; checkpoints store full tensors whatever model.TP trained them
    if device.type == "cpu":
        mcfg.model_dtype = torch.float32
    grid = ProcessGrid(world, PP=a.PP, WP_Y=a.WP_Y, WP_X=a.WP_X)
    dcfg = C.diffusion_config(cfg)
    ecfg = EngineConfig(checkpoint_dir=a.checkpoint, seed=a.seed, benchmark=True, init_policy=dict(skip=True))
    ocfg = OptimConfig(use_ema=False)
    eng = InferenceEngine(mcfg, ocfg, dcfg, ecfg, grid, rank, device, members=a.members,
                          groups={} if world == 1 else None)
    if a.checkpoint:
        assert eng.load_checkpoint(load_ema=a.load_ema, prefix=a.extra_name), f"no usable checkpoint in {a.checkpoint}"
    c = eng.c
    g = eng.ctx.grid
    C_out, C_in = mcfg.out_channels, mcfg.in_channels
    C_f = C_in - 2 * C_out
    sd = dcfg.sigma_data
    gen = torch.Generator(device=device).manual_seed(a.seed * 7919 + c.dp * 977 + c.wp_y * 31 + c.wp_x)
    rows = eng.tokens
    head = eng.is_first_stage()
    H, W = mcfg.img
    hb, wb = H // a.WP_Y, W // a.WP_X

    def to_tokens(blk):        # [..., hb, wb, C] block of this WP rank -> [..., rows, C] in the unshifted window layout
        lead = blk.shape[:-3]
        x = blk.reshape(*lead, g.nwy_loc, g.ws_y, g.nwx_loc, g.ws_x, blk.shape[-1])
        n = len(lead)
        x = x.permute(*range(n), n, n + 2, n + 1, n + 3, n + 4)
        return x.reshape(*lead, rows, blk.shape[-1])

    def to_block(tok):         # inverse of to_tokens for [M, rows, C]
        x = tok.view(tok.shape[0], g.nwy_loc, g.nwx_loc, g.ws_y, g.ws_x, tok.shape[-1]).permute(0, 1, 3, 2, 4, 5)
        return x.reshape(tok.shape[0], hb, wb, tok.shape[-1])
    data = writer = None
    if a.data:
        from ..data.inference_data import InferenceData, RolloutWriter, strided_indices
        data = InferenceData(a.data, a.data_root, (H, W), (a.WP_Y, a.WP_X), (c.wp_y, c.wp_x),
                             interval=int(cfg.model.get("interval", 6)), rollout_steps=a.rollout_steps,
                             out_channels=C_out, channels=73 if C_f > 0 else 69)
        stats = data.stats(device)
        all_ic, my_ic = strided_indices(data.ds.ds.shape[0], a.rollout_steps, data.dt, a.stride_ic, c.dp, grid.DP,
                                        start=max(a.start_sample, 0), end=None if a.end_sample < 0 else a.end_sample)
        if a.out and head:
            stem = f"output-{len(all_ic)}i-{a.rollout_steps}s-{a.members}m-{a.sampler_steps}ds{a.extra_outname}" + \
                (f"_dp{c.dp}" if grid.DP > 1 else "")
            writer = RolloutWriter(a.out, stem, (c.wp_y, c.wp_x), len(my_ic), a.rollout_steps, a.members, C_out, hb, wb)
    else:
        stats = {k: torch.zeros(C_out, device=device) if "mean" in k else torch.ones(C_out, device=device)
                 for k in ("x_mean", "x_std", "t_mean", "t_std")}
        my_ic = [0]
    ts = TF.sampler_schedule(a.sampler_steps, dcfg.sigma_min if a.sigma_min < 0 else a.sigma_min,
                             dcfg.sigma_max if a.sigma_max < 0 else a.sigma_max, sd, device=device)
    metrics = EnsembleMetrics(a.rollout_steps, C_out, H * W, device, group=eng.groups.get("wp"))
    w_lat = TF.latitude_weights(H, dcfg.w_lat_add)
    w_tok = LY.image_to_tokens(w_lat.view(1, -1, 1, 1).expand(1, H, W, 1), g, (0, 0), eng.wp_rank)
    w_tok = w_tok.to(device).view(-1)
    t0 = time.perf_counter()
    evals = 0

    def net(xs, cond, forcing, tt):
        nonlocal evals
        evals += 1
        if head:
            mi = [torch.cat([xm / sd, cm] + ([forcing] if forcing is not None else []), dim=-1)
                  for xm, cm in zip(xs, cond)]
            return eng.exec_schedule(mi, torch.tensor([tt], device=device))
        eng.exec_schedule(None, None)
        return None
    for n, idx in enumerate(my_ic):
        if data is not None:
            smp = data.sample(idx)
            state = to_tokens(smp["state"].to(device))                        # physical units, [rows, C]
            forcings = to_tokens(smp["forcing"].to(device)) if smp["forcing"] is not None else None
            truth = to_tokens(smp["truth"].to(device))
        else:
            state = torch.randn(rows, C_out, generator=gen, device=device)
            forcings = torch.randn(1, rows, C_f, generator=gen, device=device).expand(a.rollout_steps, -1, -1) if C_f > 0 else None
            truth = state.unsqueeze(0).expand(a.rollout_steps, -1, -1)
        members = [state.clone() for _ in range(a.members)]                   # physical units
        if writer is not None:
            writer.put(n, 0, to_block(torch.stack(members)))
        for k in range(a.rollout_steps):
            cond = [(m - stats["x_mean"]) / stats["x_std"] for m in members]
            forcing = forcings[k] if forcings is not None else None
            x = [torch.randn(rows, C_out, generator=gen, device=device) * sd for _ in range(a.members)]
            for i in range(a.sampler_steps):
                s_cur, tn = float(ts[i]), float(ts[i + 1])
                s, s_l = churn_rotation(s_cur, a.sampler_steps, a.S_churn, a.S_min, a.S_max)
                if s_l > 0 and head:
                    x = [math.cos(s_l) * xm + math.sin(s_l) * a.S_noise * sd *
                         torch.randn(rows, C_out, generator=gen, device=device) for xm in x]
                d = tn - s
                f_s = net(x, cond, forcing, s)
                heun = (not a.euler) and i < a.sampler_steps - 1
                if head:
                    x_e = [xm + d * sd * f for xm, f in zip(x, f_s)]
                f_t = net(x_e if head else None, cond, forcing, tn) if heun else None
                if head:
                    x = [xm + d * sd * 0.5 * (fa + fb) for xm, fa, fb in zip(x, f_s, f_t)] if heun else x_e
            if head:
                # X_{k+1} = X_k + unstandardize_t(Y) in physical units (:325-333)
                members = [m + (y * stats["t_std"] + stats["t_mean"]) for m, y in zip(members, x)]
                mem = torch.stack(members).permute(0, 2, 1).unsqueeze(-1)      # [M, C, rows, 1] "image" of token rows
                metrics.update(k, mem, truth[k].t().unsqueeze(-1), w_tok)
                if a.local_eval:
                    print0(metrics.running_line(k, 0, int(cfg.model.get("interval", 6))))
                if writer is not None:
                    writer.put(n, k + 1, to_block(torch.stack(members)))
        metrics.end_initial_condition()
    if device.type == "cuda":
        torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    if grid.DP > 1 and head and eng.groups.get("dp") is not None:    # one packed reduction over the replicas
        packed = torch.cat([metrics.err.reshape(-1), torch.tensor([float(metrics.count)], device=device, dtype=torch.float64)])
        dist.all_reduce(packed, group=eng.groups["dp"])
        metrics.err, metrics.count = packed[:-1].view_as(metrics.err), int(round(packed[-1].item()))
    agg, scores = metrics.finalize()
    if writer is not None:
        writer.close()
    if C_out in (69, 70):       # the named channel sets: scores of the nine headline variables (pp_generate.py:500-526)
        from ..data.era5 import variable_names
        print0("RMSE first member, RMSE ensemble mean, CRPS, spread/skill\n"
               + metrics.headline_table(variable_names(73)[:C_out], interval=int(cfg.model.get("interval", 6))))
    if a.out and rank == 0:
        os.makedirs(a.out, exist_ok=True)
        np.save(os.path.join(a.out, "pp_rollout_err_aggregate.npy"), agg)
        np.save(os.path.join(a.out, "pp_rollout_err.npy"), scores)
    print0(json.dumps({"entry": "pp_generate", "world": world, "PP": a.PP, "wp": [a.WP_Y, a.WP_X], "members": a.members,
                       "rollout_steps": a.rollout_steps, "network_evaluations": evals,
                       "initial_conditions": len(my_ic), "ema": bool(a.load_ema), "S_churn": a.S_churn,
                       "s_per_forecast_step": dt / max(a.rollout_steps * len(my_ic), 1)}))
    teardown()


if __name__ == "__main__":
    main()
