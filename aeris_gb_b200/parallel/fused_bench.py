"""Device-timed benchmark of the four fused compute+collective paths against their rooflines and unfused parts.

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 -m aeris_gb_b200.parallel.fused_bench

Sections (``--only tp,sp,halo,dp``): tensor-parallel MLP (all-gather -> GEMM, GEMM -> reduce-scatter), Ulysses
sequence-parallel attention (head scatter in the QKV GEMM epilogue + token-owner push in the attention epilogue),
window-parallel halo gather inside modulate+RMSNorm, and the gradient reduce-scatter + AdamW + all-gather step.
Prints one JSON line (rank 0): times are CUDA-event milliseconds per call, max over ranks, median of five batches of
``--iters`` back-to-back calls after warm-up (a batch is bracketed by a barrier and a device synchronisation).
``roofline_ms`` of a fused path is the slowest of FLOPs / ``--peak-tflops``, NVLink bytes per GPU and direction /
``--link-gbs`` and (memory-bound kernels) HBM bytes / ``--hbm-gbs``; the defaults are the measured copy bandwidth and
the measured burst cuBLAS rate of ``MEASURED_PEAKS.json`` (these kernels are timed in isolation). ``clocks`` is the
SM-clock and throttle-reason record of rank 0's GPU over the whole run.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from ..ops import gemm as G
from . import tensor as TP


def _time(fn, iters, warmup=3, batches=5):
    for _ in range(warmup):
        fn()
    ts = []
    for _ in range(batches):
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ts.append(t.item())
    ts.sort()
    return ts[len(ts) // 2]


def _measured_peaks():
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d.get("bf16_tflops", 1590.0), d.get("hbm_gbs", 6650.0), "measured", d.get("bf16_tflops_sustained", 1400.0)
    return 1590.0, 6650.0, "fallback", 1400.0


def bench_sp(a, dev, res):
    """QKV GEMM with head scatter -> barrier -> attention with token-owner push -> barrier, one 72-window chunk."""
    from ..models import fused
    from ..ops import elementwise as E
    sp = dist.get_world_size()
    D, H, d, L, nw = a.dim, 24, 64, 900, 72
    n_local = L // sp
    spx = fused.SPExchange(dist.group.WORLD, dev)
    meta = fused.BlockMeta(nw, n_local, H, d, E.MODE_MOD_THEN_NORM, 1e-3, nw, sp=spx)
    h = torch.randn(nw * n_local, D, device=dev).bfloat16()
    wqkv = (torch.randn(3 * H * d, D, device=dev) * D ** -0.5).bfloat16()
    res["sp_qkv_attn_fused_ms"] = _time(lambda: fused._sp_attention_fwd(meta, h, wqkv, nw, True), a.iters)
    flops = 2.0 * nw * n_local * D * 3 * H * d + 4.0 * nw * (H // sp) * L * L * d
    link = (sp - 1) / sp * nw * n_local * H * d * 2 * 4          # q, k, v out; o back
    res["sp_roofline_ms"] = max(flops / (a.peak_tflops * 1e9), link / (a.link_gbs * 1e6))
    # the unfused parts on one GPU: plain QKV GEMM, plain attention over this rank's heads, 4 NCCL all-to-alls
    from ..ops import attention as A
    qkv = torch.empty(nw * n_local, 3 * H * d, device=dev, dtype=torch.bfloat16)
    res["sp_qkv_gemm_local_ms"] = _time(lambda: G.gemm(h, wqkv, out=qkv), a.iters)
    qf = torch.randn(nw * L, 3 * (H // sp) * d, device=dev).bfloat16()
    of = torch.empty(nw * L, (H // sp) * d, device=dev, dtype=torch.bfloat16)
    lse = torch.empty(nw, H // sp, L, device=dev)
    res["sp_attn_local_ms"] = _time(lambda: A.attn_fwd(qf, nw, L, H // sp, d, out=of, lse=lse), a.iters)
    t_in = torch.randn(nw * n_local * H * d, device=dev).bfloat16()
    t_out = torch.empty_like(t_in)
    res["sp_nccl_all_to_all_x4_ms"] = 4 * _time(lambda: dist.all_to_all_single(t_out, t_in), a.iters)
    res["sp_frac_of_roofline"] = res["sp_roofline_ms"] / res["sp_qkv_attn_fused_ms"]
    # roofline of the compute alone, as achieved by the same kernels without any exchange
    res["sp_frac_of_unfused_compute"] = (res["sp_qkv_gemm_local_ms"] + res["sp_attn_local_ms"]) / res["sp_qkv_attn_fused_ms"]


def bench_halo(a, dev, res):
    """modulate+RMSNorm whose rows come through the shifted-window gather table from local and peer memory."""
    from ..engine.trainer import wp_grid_for
    from ..models import layout as LY
    from ..ops import elementwise as E
    from .symm import HaloExchange
    world, rank = dist.get_world_size(), dist.get_rank()
    wp = wp_grid_for(world)
    grid = LY.Grid(720, 1440, 30, 30, wp[0], wp[1])
    D = a.dim
    rows = grid.tokens_per_rank
    table = LY.gather_table(grid, (0, 0), grid.half_shift(), rank).to(dev)
    halo = HaloExchange(dist.group.WORLD, dev)
    x = torch.randn(rows, D, device=dev).bfloat16()
    peers = halo.peer_fn(x, "fwd")
    sc, sh = torch.randn(D, device=dev), torch.randn(D, device=dev)
    w = torch.ones(D, device=dev).bfloat16()
    hout, xg = torch.empty_like(x), torch.empty_like(x)

    def gathered():
        E.modnorm_fwd(None, sc, sh, w, mode=0, eps=1e-3, out=hout, gather_idx=table, peer_ptrs=peers, x_out=xg,
                      rows=rows)

    res["halo_modnorm_gather_ms"] = _time(gathered, a.iters)
    res["halo_modnorm_local_ms"] = _time(lambda: E.modnorm_fwd(x, sc, sh, w, mode=0, eps=1e-3, out=hout), a.iters)
    frac = LY.halo_fraction(grid)
    hbm = rows * D * 2 * (3 - frac)                 # read local rows, write gathered x and h
    link = frac * rows * D * 2
    res["halo_fraction"] = frac
    res["halo_roofline_ms"] = max(hbm / (a.hbm_gbs * 1e6), link / (a.link_gbs * 1e6))
    res["halo_frac_of_roofline"] = res["halo_roofline_ms"] / res["halo_modnorm_gather_ms"]
    res["halo_publish_copy_ms"] = _time(lambda: halo.peer_fn(x, "fwd"), a.iters)      # staged: copy + two barriers
    xp = halo.output_buffer(rows, D, torch.bfloat16)
    res["halo_publish_in_place_ms"] = _time(lambda: halo.peer_fn(xp, "fwd"), a.iters)   # producer wrote it there: one barrier


def bench_dp(a, dev, res):
    """Gradient reduce-scatter + clip + AdamW + bf16 all-gather over peer memory for ``--params`` parameters."""
    from ..engine.fused_dp import FusedShardedOptimizer
    from ..engine.optim import OptimConfig
    world = dist.get_world_size()
    n = a.params
    layers = torch.nn.ModuleList([torch.nn.Linear(4096, n // 4096 // 8, bias=False) for _ in range(8)]).to(dev).bfloat16()
    nparams = sum(p.numel() for p in layers.parameters())
    for mc, tag in ((False, "p2p"), (True, "multimem")):
        opt = FusedShardedOptimizer(layers, OptimConfig(grad_clip_max_norm=1.0), dist.group.WORLD, dev, use_multicast=mc)
        if mc and not opt.uses_multicast:
            res["dp_multimem"] = "multicast objects unavailable"
            continue

        def step():
            for s in opt.segments:
                s.grad.fill_(1e-3)
            opt.reduce_and_step(8, 1.0)

        def fill():
            for s in opt.segments:
                s.grad.fill_(1e-3)

        t_all = _time(step, a.iters)
        t_fill = _time(fill, a.iters)
        res[f"dp_step_{tag}_ms"] = t_all - t_fill
        link_rs = (world - 1) / world * nparams * 4
        link_ag = (world - 1) / world * nparams * 2
        # HBM bytes per rank: every gradient word is read once from this rank's memory (by itself or a peer) and
        # zeroed once; the shard reads 5 and writes 4 fp32 arrays plus the reduced gradient; every rank's bf16 shard
        # is written into this rank's parameter buffer
        hbm = nparams * 8 + nparams / world * (40 + 2 * world)
        roof = max((link_rs + link_ag) / (a.link_gbs * 1e6), hbm / (a.hbm_gbs * 1e6))
        res[f"dp_roofline_{tag}_ms"] = roof
        res[f"dp_frac_of_roofline_{tag}"] = roof / res[f"dp_step_{tag}_ms"]
        del opt
    g = torch.randn(nparams, device=dev)
    res["dp_nccl_allreduce_fp32_ms"] = _time(lambda: dist.all_reduce(g), a.iters)
    res["dp_params"] = nparams


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default="tp,sp,halo,dp")
    ap.add_argument("--params", type=int, default=1 << 29)
    ap.add_argument("--hbm-gbs", type=float, default=None)
    ap.add_argument("--rows", type=int, default=64800, help="gathered rows (all ranks)")
    ap.add_argument("--dim", type=int, default=1536)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--peak-tflops", type=float, default=None)
    ap.add_argument("--link-gbs", type=float, default=770.0)
    a = ap.parse_args()
    tf, bw, src, tf_sus = _measured_peaks()
    a.peak_tflops = a.peak_tflops or tf
    a.sustained_tflops = tf_sus
    a.hbm_gbs = a.hbm_gbs or bw
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=dev)
    res = {"world": world, "peak_tflops": a.peak_tflops, "hbm_gbs": a.hbm_gbs, "link_gbs": a.link_gbs,
           "peak_source": src}
    from ..utils.clocks import ClockSampler
    clk = ClockSampler(int(os.environ["LOCAL_RANK"]))
    clk.start()
    only = a.only.split(",")
    if "sp" in only and world in (2, 4, 8):
        bench_sp(a, dev, res)
    if "halo" in only:
        bench_halo(a, dev, res)
    if "dp" in only:
        bench_dp(a, dev, res)
    if "tp" in only:
        bench_tp(a, dev, res, rank, world)
    from ..ops import lib as L
    L.check_status()
    res["clocks"] = clk.stop()
    if rank == 0:
        print(json.dumps(res))
    dist.barrier()
    dist.destroy_process_group()


def bench_tp(a, dev, res, rank, world):
    tp = world
    n_loc = a.rows // tp
    M, D, F = n_loc * tp, a.dim, a.hidden
    tpx = TP.TPExchange(dist.group.WORLD, dev)
    w1 = (torch.randn(2 * F // tp, D, device=dev) * D ** -0.5).bfloat16()
    w2 = (torch.randn(D, F // tp, device=dev) * F ** -0.5).bfloat16()
    a_buf, peers = tpx.buffer("ag_x", (M, D))
    a_buf.normal_()
    act = torch.empty((M, F // tp), dtype=torch.bfloat16, device=dev)
    nccl_in = torch.randn(n_loc, D, device=dev).bfloat16()
    nccl_out = torch.empty((M, D), dtype=torch.bfloat16, device=dev)
    y_full = torch.empty((M, D), dtype=torch.bfloat16, device=dev)
    y_loc = torch.empty((n_loc, D), dtype=torch.bfloat16, device=dev)

    def fused_ag():
        tpx.barrier()
        TP.gemm_allgather_a(tpx, a_buf, peers, w1, out=act, epi=G.EPI_SWIGLU)

    def plain_w1():
        G.gemm(a_buf, w1, out=act, epi=G.EPI_SWIGLU, two_cta=False, bn=256)

    def plain_w1_2cta():
        G.gemm(a_buf, w1, out=act, epi=G.EPI_SWIGLU)

    def nccl_ag():
        dist.all_gather_into_tensor(nccl_out, nccl_in)

    def fused_rs():
        TP.gemm_reduce_scatter(tpx, act, w2, out=y_loc)

    def plain_w2():
        G.gemm(act, w2, out=y_full)

    def nccl_rs():
        dist.reduce_scatter_tensor(y_loc, y_full)

    res.update({"rows": M, "dim": D, "hidden": F,
           "ag_gemm_fused_ms": _time(fused_ag, a.iters), "w1_gemm_local_1cta_ms": _time(plain_w1, a.iters),
           "w1_gemm_local_2cta_ms": _time(plain_w1_2cta, a.iters), "nccl_all_gather_ms": _time(nccl_ag, a.iters),
           "gemm_rs_fused_ms": _time(fused_rs, a.iters), "w2_gemm_local_ms": _time(plain_w2, a.iters),
           "nccl_reduce_scatter_ms": _time(nccl_rs, a.iters)})
    fl1 = 2.0 * M * D * (2 * F // tp)
    fl2 = 2.0 * M * D * (F // tp)
    link = (tp - 1) / tp * M * D * 2
    res["ag_gemm_roofline_ms"] = max(fl1 / (a.peak_tflops * 1e9), link / (a.link_gbs * 1e6))
    res["gemm_rs_roofline_ms"] = max(fl2 / (a.peak_tflops * 1e9), link / (a.link_gbs * 1e6))
    res["ag_gemm_frac_of_roofline"] = res["ag_gemm_roofline_ms"] / res["ag_gemm_fused_ms"]
    res["gemm_rs_frac_of_roofline"] = res["gemm_rs_roofline_ms"] / res["gemm_rs_fused_ms"]
    # the batches run back to back for seconds, so the GPU sits at its power cap (see "clocks"): the same fractions
    # against the cuBLAS rate measured under that cap
    sus = a.sustained_tflops
    res["sustained_tflops"] = sus
    res["ag_gemm_frac_of_roofline_sustained"] = max(fl1 / (sus * 1e9), link / (a.link_gbs * 1e6)) / res["ag_gemm_fused_ms"]
    res["gemm_rs_frac_of_roofline_sustained"] = max(fl2 / (sus * 1e9), link / (a.link_gbs * 1e6)) / res["gemm_rs_fused_ms"]


if __name__ == "__main__":
    main()
