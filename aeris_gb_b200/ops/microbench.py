"""Kernel micro-benchmarks: ``python -m aeris_gb_b200.ops.microbench <gemm|attn_fwd|attn_bwd|modnorm|swiglu|adamw> ...``

Times one kernel with CUDA events (3 warm-up launches, then ``--iters`` launches, inputs larger than L2) and prints
one JSON line with achieved TFLOP/s or GB/s and, when ``MEASURED_PEAKS.json`` is present at the repository root, the
fraction of the measured cuBLAS / copy peak. Also the small fixed workload that the committed ncu summaries were
captured on.
"""
from __future__ import annotations

import argparse
import json
import os

import torch

from . import attention as A
from . import elementwise as E
from . import gemm as G
from . import lib as L


def _peaks():
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d.get("bf16_tflops", 1590.0), d.get("hbm_gbs", 6650.0), "measured"
    return 1590.0, 6650.0, "fallback"


def _time(fn, iters):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    L.check_status(sync=False)
    return e0.elapsed_time(e1) / iters


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("kernel", choices=["gemm", "attn_fwd", "attn_bwd", "modnorm", "swiglu", "adamw"])
    ap.add_argument("--m", type=int, default=32768)
    ap.add_argument("--n", type=int, default=4608)
    ap.add_argument("--k", type=int, default=1536)
    ap.add_argument("--a-t", action="store_true")
    ap.add_argument("--b-t", action="store_true")
    ap.add_argument("--epi", type=int, default=0)
    ap.add_argument("--k-splits", type=int, default=1)
    ap.add_argument("--windows", type=int, default=72)
    ap.add_argument("--tokens", type=int, default=900)
    ap.add_argument("--heads", type=int, default=24)
    ap.add_argument("--head-dim", type=int, default=64)
    ap.add_argument("--rows", type=int, default=129600)
    ap.add_argument("--dim", type=int, default=1536)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--one-cta", action="store_true", help="force the one-CTA GEMM kernel")
    a = ap.parse_args()
    dev = "cuda"
    tf_peak, bw_peak, src = _peaks()
    out = {"kernel": a.kernel}
    if a.kernel == "gemm":
        A_ = torch.randn((a.k, a.m) if a.a_t else (a.m, a.k), device=dev).bfloat16()
        B_ = torch.randn((a.k, a.n) if a.b_t else (a.n, a.k), device=dev).bfloat16()
        kw = {}
        if a.epi == G.EPI_ACC_F32:
            kw["out"] = torch.zeros(a.m, a.n, device=dev)
        if a.epi == G.EPI_GATE_RESID:
            kw["resid"] = torch.randn(a.m, a.n, device=dev).bfloat16()
            kw["gate"] = torch.randn(1, a.n, device=dev)
        ms = _time(lambda: G.gemm(A_, B_, a_t=a.a_t, b_t=a.b_t, epi=a.epi, k_splits=a.k_splits,
                                  two_cta=not a.one_cta, **kw), a.iters)
        fl = 2.0 * a.m * a.n * a.k
        out.update(shape=[a.m, a.n, a.k], a_t=a.a_t, b_t=a.b_t, epi=a.epi, ms=ms, tflops=fl / ms / 1e9,
                   frac_of_peak=fl / ms / 1e9 / tf_peak, peak_source=src)
    elif a.kernel in ("attn_fwd", "attn_bwd"):
        nw, N, H, d = a.windows, a.tokens, a.heads, a.head_dim
        qkv = torch.randn(nw * N, 3 * H * d, device=dev).bfloat16()
        o = torch.empty(nw * N, H * d, device=dev, dtype=torch.bfloat16)
        lse = torch.empty(nw, H, N, device=dev)
        A.attn_fwd(qkv, nw, N, H, d, out=o, lse=lse)
        if a.kernel == "attn_fwd":
            ms = _time(lambda: A.attn_fwd(qkv, nw, N, H, d, out=o, lse=lse), a.iters)
            fl = 4.0 * nw * H * N * N * d
        else:
            go = torch.randn_like(o)
            dq = torch.empty_like(qkv)
            delta = torch.empty_like(lse)
            ms = _time(lambda: A.attn_bwd(qkv, o, go, lse, nw, N, H, d, dqkv=dq, delta=delta), a.iters)
            fl = 10.0 * nw * H * N * N * d
        out.update(shape=[nw, N, H, d], ms=ms, tflops=fl / ms / 1e9, frac_of_peak=fl / ms / 1e9 / tf_peak,
                   peak_source=src)
    elif a.kernel == "modnorm":
        x = torch.randn(a.rows, a.dim, device=dev).bfloat16()
        sc, sh = torch.randn(a.dim, device=dev), torch.randn(a.dim, device=dev)
        w = torch.ones(a.dim, device=dev).bfloat16()
        h = torch.empty_like(x)
        ms = _time(lambda: E.modnorm_fwd(x, sc, sh, w, mode=0, eps=1e-3, out=h), a.iters)
        by = 2.0 * x.numel() * 2
        out.update(shape=[a.rows, a.dim], ms=ms, gbs=by / ms / 1e6, frac_of_peak=by / ms / 1e6 / bw_peak,
                   peak_source=src)
    elif a.kernel == "swiglu":
        u = torch.randn(a.rows, 2 * a.dim, device=dev).bfloat16()
        act = torch.empty(a.rows, a.dim, device=dev, dtype=torch.bfloat16)
        ms = _time(lambda: E.swiglu_fwd(u, out=act), a.iters)
        by = 3.0 * a.rows * a.dim * 2
        out.update(shape=[a.rows, a.dim], ms=ms, gbs=by / ms / 1e6, frac_of_peak=by / ms / 1e6 / bw_peak,
                   peak_source=src)
    else:
        n = a.rows * a.dim
        bufs = [torch.randn(n, device=dev) for _ in range(5)]
        wb = torch.empty(n, device=dev, dtype=torch.bfloat16)
        ms = _time(lambda: E.adamw(bufs[0], bufs[1], bufs[2].abs_(), bufs[3].abs_(), wb, bufs[4], None, lr=1e-4,
                                   betas=(0.9, 0.99), eps=1e-8, weight_decay=0.0, step=3, grad_scale=1.0,
                                   max_norm=0.0, ema_beta=0.999), a.iters)
        by = n * (5 * 4 + 5 * 4 + 2.0)
        out.update(n=n, ms=ms, gbs=by / ms / 1e6, frac_of_peak=by / ms / 1e6 / bw_peak, peak_source=src)
    print(json.dumps(out))


if __name__ == "__main__":
    main()
