#!/usr/bin/env python
"""Headline benchmark: TrigFlow training throughput of the ~1.3B-class AERIS Swin diffusion model at 720x1440.

    python bench.py --gpus N --steps K --warmup W            (N > 1: launched once per rank by torch.distributed.run)

Weak scaling: the global batch is N samples; every sample is window-parallel over all N GPUs (WP = N), so each GPU
always holds 1,036,800 tokens per step. Synthetic N(0,1) fields, random-init weights, bf16 compute with fp32 master
weights, full optimizer step inside the timed region. Prints ONE JSON line on rank 0.

Other arms: ``--impl reference`` (the unmodified reference modules on stock PyTorch kernels, data parallel), ``--impl torch-eager`` (the same model
through stock PyTorch ops, an informational same-math baseline), ``--mode infer`` (seconds per autoregressive forecast
step, one ensemble member per GPU), ``--sp S`` (WP = N / S with Ulysses sequence parallelism S), ``--tp T`` (MLP weights
split over the SP group, or over all ranks without SP).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
# the flagship run fills most of the 180 GB; growable segments keep the caching allocator from fragmenting it
os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")


FLAGSHIP = {   # plain numbers shared by both arms (no package import needed to read them)
    "full": dict(img=(720, 1440), window=(30, 30), dim=1536, heads=24, head_dim=64, mlp_dim=4096, n_layers=40,
                 in_ch=144, out_ch=70, chunk_windows=72),
    "quarter": dict(img=(360, 720), window=(30, 30), dim=1536, heads=24, head_dim=64, mlp_dim=4096, n_layers=10,
                    in_ch=144, out_ch=70, chunk_windows=72),
    "tiny": dict(img=(120, 240), window=(30, 30), dim=256, heads=4, head_dim=64, mlp_dim=512, n_layers=4,
                 in_ch=144, out_ch=70, chunk_windows=8),
}
METRIC_TRAIN = "train samples/s (TrigFlow, 720x1440 Swin diffusion)"
METRIC_INFER = "WP-infer s/step (one member per GPU)"


def model_label(d: dict) -> str:
    return (f"AERIS Swin TrigFlow dim{d['dim']} x{d['n_layers']} blocks heads{d['heads']}x{d['head_dim']} "
            f"mlp{d['mlp_dim']} window{d['window'][0]}x{d['window'][1]} channels{d['in_ch']}->{d['out_ch']}")


def reference_arm(args):
    """The unmodified reference modules (a copy of the reference's ``src/`` under ``baseline/_ref``) driven by
    ``baseline/harness.py`` on stock PyTorch kernels: data parallel over the N GPUs, one full sample per GPU, so global
    batch and tokens per GPU equal the framework's run. Nothing of ``aeris_gb_b200`` is imported on this path.
    One pass of K steps gives both numbers: every step copies its inputs from pinned host memory and reads the loss
    back (end to end); CUDA events after the copy and before the read-back give the device-only time."""
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from baseline import harness as HN
    why = HN.reference_available()
    if why:
        print(json.dumps({"impl": "reference", "unavailable": why}))
        return 0
    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29517")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    d = dict(FLAGSHIP[args.scale])
    if args.layers:
        d["n_layers"] = args.layers
    if args.chunk_windows:
        d["chunk_windows"] = args.chunk_windows
    H, Wd = d["img"]
    W, K = max(args.warmup, 3), args.steps
    gen = torch.Generator().manual_seed(100 + rank)

    def sync_all():
        dist.barrier()
        torch.cuda.synchronize()

    if args.mode == "infer":
        fc = HN.ReferenceForecaster(d, dev, sampler_steps=args.sampler_steps, seed=rank)
        g7 = torch.Generator().manual_seed(7)
        state = torch.randn(1, H * Wd, d["out_ch"], generator=g7).to(dev)
        forcing = torch.randn(1, H * Wd, d["in_ch"] - 2 * d["out_ch"], generator=g7).to(dev)
        warm = HN.ReferenceForecaster.__new__(HN.ReferenceForecaster)      # same model, two sampler steps
        warm.__dict__.update(fc.__dict__)
        warm.n = min(2, args.sampler_steps)
        warm.t_steps = fc.t_steps[[0, -2, -1]] if fc.n > 2 else fc.t_steps
        state = warm.step(state, forcing)
        sync_all()
        clk = ClockSampler(local_rank)
        clk.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(K):
            state = fc.step(state, forcing)
        e1.record()
        sync_all()
        t = torch.tensor([e0.elapsed_time(e1) / 1e3 / K], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        clocks = clk.stop()
        if rank == 0:
            n_par = sum(p.numel() for p in fc.model.parameters())
            print(json.dumps({
                "impl": "reference", "metric": METRIC_INFER, "value": t.item(), "unit": "s per forecast step",
                "n_gpus": world, "steps": K, "warmup": 1, "higher_is_better": False, "scaling": "weak",
                "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "members": world,
                "config": {"model": model_label(d), "params": n_par, "sampler_steps": args.sampler_steps,
                           "network_evals_per_step": 2 * args.sampler_steps - 1, "scale": args.scale,
                           "state_finite": bool(torch.isfinite(state).all().item())},
                "clocks": clocks, "peak_mem_gb": torch.cuda.max_memory_allocated() / 1e9}))
        dist.destroy_process_group()
        return 0

    tr = HN.ReferenceTrainer(d, dev, group=dist.group.WORLD)
    host = [(torch.randn(1, H, Wd, d["out_ch"], generator=gen).pin_memory(),
             torch.randn(1, H, Wd, d["in_ch"] - d["out_ch"], generator=gen).pin_memory()) for _ in range(2)]
    h2d = sum(t_.numel() * 4 for t_ in host[0])
    for i in range(W):
        tr.train_step(*host[i % 2])
    sync_all()
    clk = ClockSampler(local_rank)
    clk.start()
    marks = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(K)]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record()
    loss = None
    for i in range(K):
        loss = tr.train_step(*host[i % 2], marks=marks[i])
    e1.record()
    sync_all()
    wall = (time.perf_counter() - t0) * 1e3
    ms_dev = sum(a.elapsed_time(b) for a, b in marks)
    tt = torch.tensor([ms_dev, max(e0.elapsed_time(e1), wall)], device=dev, dtype=torch.float64)
    dist.all_reduce(tt, op=dist.ReduceOp.MAX)
    clocks = clk.stop()
    ms_dev, ms_e = tt[0].item() / K, tt[1].item() / K
    B = world
    if rank == 0:
        print(json.dumps({
            "impl": "reference", "metric": METRIC_TRAIN, "value": B / (ms_dev / 1e3), "unit": "samples/s",
            "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": ms_dev, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "tflops_per_gpu": tr.flops_per_step(B) / (ms_dev / 1e3) / 1e12 / world,
            "config": {"model": model_label(d), "params": tr.param_count, "global_batch": B, "seq_len": H * Wd,
                       "parallelism": f"dp{world}", "scale": args.scale,
                       "activation_checkpointing": "per layer and window chunk (harness glue)",
                       "l2": "inputs (597 MB/step/GPU) and activations are far larger than L2",
                       "timing": "one pass: device time between events after the H2D copy and before the loss read"},
            "clocks": clocks,
            "e2e": {"value": B / (ms_e / 1e3), "unit": "samples/s", "ms_per_step": ms_e, "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": 4, "last_loss": loss},
            "peak_mem_gb": torch.cuda.max_memory_allocated() / 1e9}))
    dist.destroy_process_group()
    return 0


def _load_clock_sampler():
    # by file path: the reference arm must not import the aeris_gb_b200 package, and this module needs none of it
    import importlib.util
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "aeris_gb_b200", "utils", "clocks.py")
    spec = importlib.util.spec_from_file_location("_aeris_clocks", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.ClockSampler


ClockSampler = _load_clock_sampler()


def flagship_config(n_gpus: int, scale: str, sp: int = 1):
    from aeris_gb_b200.engine.trainer import wp_grid_for
    from aeris_gb_b200.models.aeris import AerisConfig
    d = FLAGSHIP[scale]
    return AerisConfig(img=d["img"], window=d["window"], in_channels=d["in_ch"], out_channels=d["out_ch"],
                       dim=d["dim"], heads=d["heads"], head_dim=d["head_dim"], mlp_dim=d["mlp_dim"],
                       n_layers=d["n_layers"], sublayers=1, wp=wp_grid_for(n_gpus // sp), sp=sp,
                       chunk_windows=d["chunk_windows"])


def infer_arm(args):
    """WP-only ensemble forecast, one member per GPU: seconds per 6-hour forecast step (``--sampler-steps`` TrigFlow
    steps, Heun on all but the last: 2 n - 1 network evaluations), device-timed, max over ranks. ``--steps`` forecast
    steps are timed after a short warm-up forecast step (three network evaluations)."""
    import torch
    import torch.distributed as dist
    from aeris_gb_b200.diffusion.rollout import DeviceForecaster, SamplerConfig
    from aeris_gb_b200.models.aeris import AerisModel, StreamContext
    from aeris_gb_b200.ops import lib as L

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    cfg = flagship_config(1, args.scale)              # every GPU holds the whole image of its member
    if args.layers:
        cfg.n_layers = args.layers
    torch.manual_seed(0)
    model = AerisModel(cfg).to(dev).eval()
    C = cfg.out_channels
    stats = {"x_mean": torch.zeros(C, device=dev), "x_std": torch.ones(C, device=dev),
             "t_mean": torch.zeros(C, device=dev), "t_std": torch.ones(C, device=dev)}
    sampler = SamplerConfig(n_steps=args.sampler_steps, heun=True)
    fc = DeviceForecaster(model, StreamContext(cfg, 1), stats, sampler, C, seed=1, member0=rank)
    gen = torch.Generator().manual_seed(7)            # the same initial state for every member, noise differs
    state = torch.randn(1, cfg.img[0], cfg.img[1], C, generator=gen).to(dev)
    forcing = torch.randn(1, cfg.img[0], cfg.img[1], cfg.in_channels - 2 * C, generator=gen).to(dev)
    # warm-up: a short forecast step (two sampler steps = three network evaluations through every kernel)
    warm = DeviceForecaster(model, StreamContext(cfg, 1), stats, SamplerConfig(n_steps=min(2, args.sampler_steps), heun=True),
                            C, seed=2, member0=rank)
    state = warm.step(state, forcing)
    del warm
    L.check_status()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    clk = ClockSampler(local_rank)
    clk.start()
    l0 = L.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        state = fc.step(state, forcing)
    e1.record()
    torch.cuda.synchronize()
    L.check_status(sync=False)
    t = torch.tensor([e0.elapsed_time(e1) / 1e3 / args.steps], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    clocks = clk.stop()
    if rank == 0:
        print(json.dumps({
            "metric": METRIC_INFER, "value": t.item(), "unit": "s per forecast step",
            "n_gpus": world, "steps": args.steps, "warmup": 1, "higher_is_better": False, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "members": world,
            "member_forecast_steps_per_s": world / t.item(),
            "config": {"model": model_label({**FLAGSHIP[args.scale], "n_layers": cfg.n_layers}),
                       "params": cfg.param_count(), "sampler_steps": args.sampler_steps, "network_evals_per_step": fc.model_evals_per_forecast_step(),
                       "scale": args.scale, "state_finite": bool(torch.isfinite(state).all().item())},
            "clocks": clocks, "gpu_launches": L.launch_count() - l0, "peak_mem_gb": torch.cuda.max_memory_allocated() / 1e9}))
    if world > 1:
        dist.destroy_process_group()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "torch-eager"],
                    help="torch-eager: the same model through stock PyTorch ops (cuBLAS, SDPA) with per-block "
                         "checkpointing: an informational same-math baseline, not the reference arm")
    ap.add_argument("--scale", default="full", choices=["full", "quarter", "tiny"])
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--layers", type=int, default=0, help="override the number of Swin layers (development only)")
    ap.add_argument("--chunk-windows", type=int, default=0)
    ap.add_argument("--sp", type=int, default=1, help="Ulysses sequence-parallel degree (WP = gpus / sp)")
    ap.add_argument("--tp", type=int, default=1,
                    help="tensor-parallel MLP degree: the SP group when --sp > 1, else all WP ranks (must equal its size)")
    ap.add_argument("--phases", type=int, default=0,
                    help="after the timed steps, run this many more with device timers around the phases of a step "
                         "(load, fwd, bwd, reduce_step, halo_barrier) and print their milliseconds per step, max over ranks")
    ap.add_argument("--mode", default="train", choices=["train", "infer"],
                    help="infer: one autoregressive forecast step per member, one member per GPU (s/step)")
    ap.add_argument("--sampler-steps", type=int, default=10)
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    if args.mode == "infer":
        return infer_arm(args)

    import torch
    import torch.distributed as dist
    from aeris_gb_b200.engine.optim import OptimConfig
    from aeris_gb_b200.engine.trainer import DiffusionConfig, Trainer
    from aeris_gb_b200.ops import lib as L

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    group = None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        group = dist.group.WORLD

    eager = args.impl == "torch-eager"
    parity = None
    if world > 1 and not eager:
        # outside the timed region: the multi-GPU kernels of this run against one GPU on a small model
        from aeris_gb_b200.parallel.parity import wp_parity
        parity = wp_parity(dev, args.sp)
        if parity["max_rel_err"] > 3e-2:
            raise SystemExit(f"multi-GPU parity check failed: {parity}")
    cfg = flagship_config(world, args.scale, args.sp)
    if eager:
        os.environ["AERIS_FORCE_ORACLE"] = "1"
        cfg.oracle_checkpoint = True
    if args.layers:
        cfg.n_layers = args.layers
    if args.chunk_windows:
        cfg.chunk_windows = args.chunk_windows
    W = max(args.warmup, 3)
    K = args.steps
    B = world                                   # global batch N, every sample split over the N WP ranks
    sp_group = None
    if args.sp > 1:
        for r0 in range(0, world, args.sp):     # consecutive ranks share windows (sp is the fastest grid axis)
            g_ = dist.new_group(list(range(r0, r0 + args.sp)))
            if r0 <= rank < r0 + args.sp:
                sp_group = g_
    tp_kw = {}
    if args.tp > 1:
        # the tensor-parallel group: the SP group, or every rank when there is no SP; the ranks holding the same shard
        tp_size = args.sp if args.sp > 1 else world
        assert args.tp == tp_size, f"--tp must be {tp_size} in this layout"
        cfg.tp, cfg.tp_rank = args.tp, rank % args.tp
        if tp_size < world:
            for pos in range(tp_size):
                g_ = dist.new_group(list(range(pos, world, tp_size)))
                if rank % tp_size == pos:
                    tp_kw["tp_ortho_group"] = g_
    trainer = Trainer(cfg, OptimConfig(), DiffusionConfig(), dev, wp_group=group, sp_group=sp_group, **tp_kw,
                      **(dict(fused_io=False, fused_dp=False) if eager else {}))
    g = cfg.grid()
    hb, wb = cfg.img[0] // cfg.wp[0], cfg.img[1] // cfg.wp[1]
    gen = torch.Generator().manual_seed(100 + rank)
    host = []
    for i in range(2):   # two different synthetic batches in pinned host memory, used alternately
        host.append((torch.randn(B, hb, wb, cfg.out_channels, generator=gen).pin_memory(),
                     torch.randn(B, hb, wb, 74, generator=gen).pin_memory()))
    devb = [(a.to(dev), b.to(dev)) for a, b in host]
    h2d = host[0][0].numel() * 4 + host[0][1].numel() * 4

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def step_device(i):
        trainer.train_step(*devb[i % 2], read_loss=False)

    def step_e2e(i):
        return trainer.train_step(*host[i % 2], read_loss=True)

    for i in range(W):
        step_device(i)
    L.check_status()

    def timed(fn, n):
        sync_all()
        sampler = ClockSampler(local_rank)
        sampler.start()
        l0 = L.launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        e0.record()
        out = None
        for i in range(n):
            out = fn(i)
        e1.record()
        sync_all()
        wall = time.perf_counter() - t0
        ms = e0.elapsed_time(e1)
        clocks = sampler.stop()
        tt = torch.tensor([ms, wall * 1e3], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        return tt[0].item() / n, tt[1].item() / n, clocks, L.launch_count() - l0, out

    ms_dev, _, clocks, launches, _ = timed(step_device, K)
    e2e = None
    if not args.no_e2e:
        ms_e, wall_e, _, _, loss = timed(step_e2e, K)
        ms_e = max(ms_e, wall_e)
        e2e = {"value": B / (ms_e / 1e3), "unit": "samples/s", "ms_per_step": ms_e, "h2d_bytes_per_step": h2d,
               "d2h_bytes_per_step": 4, "last_loss": loss}
    L.check_status()
    phases = None
    if args.phases > 0:
        trainer.timers.enabled = True
        trainer.timers.use_nvtx = False
        sync_all()
        for i in range(args.phases):
            step_device(i)
        phases = {k: v / args.phases for k, v in trainer.timers.resolve().items()}
        trainer.timers.enabled = False
    flops = trainer.flops_per_step(B)
    if rank == 0:
        out = {
            **({"impl": "torch-eager"} if eager else {}),
            "metric": METRIC_TRAIN, "value": B / (ms_dev / 1e3),
            "unit": "samples/s", "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": ms_dev,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "tflops_per_gpu": flops / (ms_dev / 1e3) / 1e12 / world,
            "config": {"model": model_label({**FLAGSHIP[args.scale], "n_layers": cfg.n_layers}),
                       "params": cfg.param_count(), "global_batch": B, "seq_len": cfg.img[0] * cfg.img[1], "parallelism": f"wp{world // args.sp}" + (f"xsp{args.sp}" if args.sp > 1 else "")
                       + (f"xtp{args.tp}(mlp)" if args.tp > 1 else ""),
                       "scale": args.scale, "activation_checkpointing": "per block",
                       "l2": "inputs (597 MB/step/GPU) and activations are far larger than L2"},
            "clocks": clocks, "gpu_launches": launches, "e2e": e2e, "parity": parity,
            "peak_mem_gb": torch.cuda.max_memory_allocated() / 1e9,
            **({"phases_ms_per_step": phases} if phases else {}),
        }
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
