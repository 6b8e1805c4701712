"""Device-timed benchmark of the fused tensor-parallel GEMMs against their unfused parts.

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 -m aeris_gb_b200.parallel.tp_bench

Prints one JSON line (rank 0): times are CUDA-event milliseconds, max over ranks, median of ``--iters`` runs after
warm-up. ``roofline_ms`` of a fused kernel is the slower of FLOPs / ``--peak-tflops`` and NVLink bytes / ``--link-gbs``.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from ..ops import gemm as G
from . import tensor as TP


def _time(fn, iters, warmup=3):
    for _ in range(warmup):
        fn()
    ts = []
    for _ in range(iters):
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1)], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ts.append(t.item())
    ts.sort()
    return ts[len(ts) // 2]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=64800, help="gathered rows (all ranks)")
    ap.add_argument("--dim", type=int, default=1536)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--peak-tflops", type=float, default=1406.8)
    ap.add_argument("--link-gbs", type=float, default=770.0)
    a = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=dev)
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

    res = {"world": world, "rows": M, "dim": D, "hidden": F,
           "ag_gemm_fused_ms": _time(fused_ag, a.iters), "w1_gemm_local_1cta_ms": _time(plain_w1, a.iters),
           "w1_gemm_local_2cta_ms": _time(plain_w1_2cta, a.iters), "nccl_all_gather_ms": _time(nccl_ag, a.iters),
           "gemm_rs_fused_ms": _time(fused_rs, a.iters), "w2_gemm_local_ms": _time(plain_w2, a.iters),
           "nccl_reduce_scatter_ms": _time(nccl_rs, a.iters)}
    fl1 = 2.0 * M * D * (2 * F // tp)
    fl2 = 2.0 * M * D * (F // tp)
    link = (tp - 1) / tp * M * D * 2
    res["ag_gemm_roofline_ms"] = max(fl1 / (a.peak_tflops * 1e9), link / (a.link_gbs * 1e6))
    res["gemm_rs_roofline_ms"] = max(fl2 / (a.peak_tflops * 1e9), link / (a.link_gbs * 1e6))
    res["ag_gemm_frac_of_roofline"] = res["ag_gemm_roofline_ms"] / res["ag_gemm_fused_ms"]
    res["gemm_rs_frac_of_roofline"] = res["gemm_rs_roofline_ms"] / res["gemm_rs_fused_ms"]
    from ..ops import lib as L
    L.check_status()
    if rank == 0:
        print(json.dumps(res))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
