"""Pipeline-parallel ensemble inference with on-the-fly scores.

    torchrun --nproc-per-node 8 -m aeris_gb_b200.cli.pp_generate --checkpoint DIR --PP 2 --WP-Y 1 --WP-X 2 --members 4

Reference: src/aeris/pp_generate.py (CLI :28-53, rollout :62-526, sampler :113-119/:298-322, metrics :346-472, output
files :93-99/:486-496). The sampler runs on the first pipeline stage and pushes every network evaluation through the
pipeline with the ensemble members as micro-batches; the autoregressive state stays on the device. Without
``--checkpoint`` random weights and synthetic N(0,1) fields are used.
"""
from __future__ import annotations

import argparse
import json
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
    ap.add_argument("--rollout-steps", type=int, default=2)
    ap.add_argument("--sampler-steps", type=int, default=20)
    ap.add_argument("--S-churn", type=float, default=0.0)
    ap.add_argument("--euler", action="store_true")
    ap.add_argument("--load-ema", action="store_true")
    ap.add_argument("--out", default=None)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("overrides", nargs="*")
    return ap.parse_args(argv)


def main(argv=None):
    a = parse(argv)
    rank, world, device = setup()
    if a.checkpoint and os.path.exists(os.path.join(a.checkpoint, ".hydra", "config.yaml")):
        cfg = C.load_run_config(a.checkpoint)
    else:
        cfg = C.compose("train", [f"experiment={a.experiment}"] + list(a.overrides))
    cfg.model.WP_Y, cfg.model.WP_X = a.WP_Y, a.WP_X
    mcfg = C.model_config(cfg)
    if device.type == "cpu":
        mcfg.model_dtype = torch.float32
    grid = ProcessGrid(world, PP=a.PP, WP_Y=a.WP_Y, WP_X=a.WP_X)
    dcfg = C.diffusion_config(cfg)
    ecfg = EngineConfig(checkpoint_dir=a.checkpoint, seed=a.seed, benchmark=True, init_policy=dict(skip=True))
    ocfg = OptimConfig(use_ema=False)
    eng = InferenceEngine(mcfg, ocfg, dcfg, ecfg, grid, rank, device, members=a.members,
                          groups={} if world == 1 else None)
    if a.checkpoint:
        eng.load_checkpoint()
    c = eng.c
    g = eng.ctx.grid
    C_out, C_in = mcfg.out_channels, mcfg.in_channels
    C_f = C_in - 2 * C_out
    sd = dcfg.sigma_data
    gen = torch.Generator(device=device).manual_seed(a.seed * 7919 + c.wp_y * 31 + c.wp_x)
    rows = eng.tokens
    head = eng.is_first_stage()
    state = torch.randn(rows, C_out, generator=gen, device=device)           # standardised synthetic initial state
    members = [state.clone() for _ in range(a.members)]
    forcing = torch.randn(rows, C_f, generator=gen, device=device) if C_f > 0 else None
    ts = TF.sampler_schedule(a.sampler_steps, dcfg.sigma_min, dcfg.sigma_max, sd, device=device)
    metrics = EnsembleMetrics(a.rollout_steps, C_out, mcfg.img[0] * mcfg.img[1], device, group=eng.groups.get("wp"))
    w_lat = TF.latitude_weights(mcfg.img[0], dcfg.w_lat_add)
    w_tok = LY.image_to_tokens(w_lat.view(1, -1, 1, 1).expand(1, mcfg.img[0], mcfg.img[1], 1), g, (0, 0), eng.wp_rank)
    w_tok = w_tok.to(device).view(-1)
    t0 = time.perf_counter()
    evals = 0
    for k in range(a.rollout_steps):
        x = [torch.randn(rows, C_out, generator=gen, device=device) * sd for _ in range(a.members)]
        for i in range(a.sampler_steps):
            s, tn = float(ts[i]), float(ts[i + 1])
            d = tn - s

            def net(xs, tt):
                nonlocal evals
                evals += 1
                if head:
                    mi = [torch.cat([xm / sd, cm] + ([forcing] if forcing is not None else []), dim=-1)
                          for xm, cm in zip(xs, members)]
                    return eng.exec_schedule(mi, torch.tensor([tt], device=device))
                eng.exec_schedule(None, None)
                return None
            f_s = net(x, s)
            heun = (not a.euler) and i < a.sampler_steps - 1
            if head:
                x_e = [xm + d * sd * f for xm, f in zip(x, f_s)]
            f_t = net(x_e if head else None, tn) if heun else None
            if head:
                x = [xm + d * sd * 0.5 * (fa + fb) for xm, fa, fb in zip(x, f_s, f_t)] if heun else x_e
        if head:
            members = [m + y for m, y in zip(members, x)]        # residual add (statistics are identity here)
            mem = torch.stack(members).permute(0, 2, 1).unsqueeze(-1)      # [M, C, rows, 1] "image" of token rows
            metrics.update(k, mem, state.t().unsqueeze(-1), w_tok)
    if device.type == "cuda":
        torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    metrics.end_initial_condition()
    agg, scores = metrics.finalize()
    if a.out and rank == 0:
        os.makedirs(a.out, exist_ok=True)
        np.save(os.path.join(a.out, "pp_rollout_err_aggregate.npy"), agg)
        np.save(os.path.join(a.out, "pp_rollout_err.npy"), scores)
    print0(json.dumps({"entry": "pp_generate", "world": world, "PP": a.PP, "wp": [a.WP_Y, a.WP_X], "members": a.members,
                       "rollout_steps": a.rollout_steps, "network_evaluations": evals,
                       "s_per_forecast_step": dt / max(a.rollout_steps, 1)}))
    teardown()


if __name__ == "__main__":
    main()
