"""Self-check of the multi-GPU paths: a small model run window-parallel (and sequence-parallel) over the ranks of the
current process group has to reproduce the same model run on one GPU, outputs and weight gradients.

Used by ``tests/wp_worker.py`` (the multi-GPU parity tests) and by ``bench.py`` before its warm-up, so that every
multi-GPU benchmark line carries the measured deviation of the very kernels it times (halo pull inside
modulate+norm, Ulysses head scatter in the QKV epilogue, attention pushes).
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def _rel(a: torch.Tensor, b: torch.Tensor) -> float:
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12)).item()


def wp_parity(device, sp: int = 1, verbose: bool = False) -> dict:
    """Collective over the default process group (one rank per GPU). Returns ``{"max_rel_err", "out_rel_err", "n",
    "wp", "sp", "worst"}``; the relative errors are maxima over ranks."""
    from ..engine.trainer import wp_grid_for
    from ..models import layout as LY
    from ..models.aeris import AerisConfig, AerisModel, StreamContext
    from ..ops import lib as L
    from .symm import HaloExchange
    rank, world = dist.get_rank(), dist.get_world_size()
    wp = wp_grid_for(world // sp)
    base = dict(img=(64, 128), window=(16, 16), in_channels=12, out_channels=6, dim=256, heads=4, head_dim=64,
                mlp_dim=256, n_layers=3, sublayers=1, norm_eps=1e-3, chunk_windows=3)
    B = 2
    torch.manual_seed(7)
    ref = AerisModel(AerisConfig(**base)).to(device)
    for n, p in ref.named_parameters():
        if "modulation" in n and p.dim() == 2:
            torch.nn.init.normal_(p, std=0.05)
    par = AerisModel(AerisConfig(**base, wp=wp, sp=sp)).to(device)
    par.load_state_dict(ref.state_dict())
    g = torch.Generator(device="cpu").manual_seed(3)
    x = torch.randn(B, 64, 128, 12, generator=g).to(device)
    r = torch.randn(B, 64, 128, 6, generator=g).to(device)
    t = torch.tensor([0.4, 1.1], device=device)
    y_ref = ref(x, t)                                   # (a) one rank, whole image
    (y_ref * r).sum().backward()
    cfg = par.cfg                                       # (b) window / sequence parallel on this rank's block
    grid = cfg.grid()
    halo = HaloExchange(dist.group.WORLD, device)
    ctx = StreamContext(cfg, B, rank, halo.peer_fn)
    if sp > 1:
        from ..models.fused import SPExchange
        sp_group = None
        for r0 in range(0, world, sp):                  # consecutive ranks form an SP group (sp is the fastest axis)
            g_ = dist.new_group(list(range(r0, r0 + sp)))
            if r0 <= rank < r0 + sp:
                sp_group = g_
        ctx.sp_group = sp_group
        ctx.sp_exchange = SPExchange(sp_group, device)
    tok = LY.image_to_tokens(x, grid, (0, 0), rank)
    rt = LY.image_to_tokens(r, grid, (0, 0), rank)
    y = par.forward_tokens(tok, t, ctx)
    (y * rt).sum().backward()
    y_ref_tok = LY.image_to_tokens(y_ref.detach(), grid, (0, 0), rank)
    errs = {"out": _rel(y.detach(), y_ref_tok)}
    for (n, p), (_, q) in zip(par.named_parameters(), ref.named_parameters()):
        if p.grad is None or q.grad is None or q.grad.float().norm() == 0:
            continue
        gsum = p.grad.float().clone()
        dist.all_reduce(gsum)
        errs[n] = _rel(gsum, q.grad)
    L.check_status()
    worst_key = max(errs, key=errs.get)
    flag = torch.tensor([errs[worst_key], errs["out"]], device=device)
    dist.all_reduce(flag, op=dist.ReduceOp.MAX)
    out = {"max_rel_err": flag[0].item(), "out_rel_err": flag[1].item(), "n": world, "wp": list(wp), "sp": sp,
           "worst": worst_key}
    if verbose and rank == 0:
        bad = {k: v for k, v in errs.items() if v > 3e-2}
        print(f"wp={wp} sp={sp} worst rel err {out['max_rel_err']:.4f} out {out['out_rel_err']:.5f} bad={bad}", flush=True)
    del halo, ctx, par, ref
    torch.cuda.empty_cache()
    return out
