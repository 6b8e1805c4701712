"""Kernel micro-benchmarks: ``python -m aeris_gb_b200.ops.microbench <gemm|attn_fwd|attn_bwd|modnorm|modnorm_bwd|swiglu|adamw|embed|loss> ...``

Times one kernel with CUDA events (3 warm-up launches, then ``--iters`` launches, inputs larger than L2) and prints
one JSON line with achieved TFLOP/s or GB/s and, when ``MEASURED_PEAKS.json`` is present at the repository root, the
fraction of the measured cuBLAS / copy peak. Also the small fixed workload that the committed ncu summaries were
captured on.

The ``fused_*`` kernels are the compute+collective kernels run on ONE GPU with the second rank's buffers placed in the
same GPU's memory (``peers`` = two local buffers): the same code path, instruction mix and tile pipeline as in a
multi-GPU run, minus the NVLink latency, which is what a single-process profiler capture can show. Their multi-GPU
timings come from ``aeris_gb_b200.parallel.fused_bench``.
"""
from __future__ import annotations

import argparse
import json
import os

import torch

from ..utils.clocks import ClockSampler
from . import attention as A
from . import elementwise as E
from . import gemm as G
from . import lib as L

_CLOCKS: list = []      # one record per timed region of this process


def _peaks():
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d.get("bf16_tflops", 1590.0), d.get("hbm_gbs", 6650.0), "measured"
    return 1590.0, 6650.0, "fallback"


def _time(fn, iters):
    """Mean milliseconds per launch: 3 warm-up launches, then at least ``iters`` launches and at least ~0.8 s of them,
    so that the clock sampler (one sample per 200 ms) sees the kernel under load."""
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    fn()
    e1.record()
    torch.cuda.synchronize()
    iters = max(iters, min(20000, int(800.0 / max(e0.elapsed_time(e1), 1e-3))))
    clk = ClockSampler(torch.cuda.current_device())
    clk.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    _CLOCKS.append(clk.stop())
    L.check_status(sync=False)
    return e0.elapsed_time(e1) / iters


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("kernel", choices=["gemm", "attn_fwd", "attn_bwd", "modnorm", "modnorm_bwd", "swiglu", "adamw",
                                       "embed", "loss", "fused_ag_gemm", "fused_rs_gemm", "fused_scatter_heads",
                                       "fused_grad_rs", "fused_shard_adamw", "fused_modnorm_gather"])
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
    ap.add_argument("--fwd-variant", type=int, default=None,
                    help="attn_fwd: softmax arithmetic of the head_dim-64 kernel (-1, 0, 2; see ops.attention)")
    ap.add_argument("--fwd-mode", type=int, default=0, help="attn_fwd: kernel mode 0..2 (see ops.attention.set_fwd_variant)")
    ap.add_argument("--smem-pad", type=int, default=0, help="attn_fwd: extra shared memory per CTA (fewer CTAs per SM)")
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
        if a.epi == G.EPI_SWIGLU_BOTH:
            kw["aux"] = torch.empty(a.m, a.n, device=dev, dtype=torch.bfloat16)
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
        if a.fwd_variant is not None or a.fwd_mode:
            A.set_fwd_variant(a.fwd_variant if a.fwd_variant is not None else -1, a.fwd_mode)
            out["fwd_variant"], out["fwd_mode"] = a.fwd_variant, a.fwd_mode
        if a.smem_pad:
            L.lib().aeris_attn_set_fwd_smem_pad(a.smem_pad)
            out["smem_pad"] = a.smem_pad
        A.attn_fwd(qkv, nw, N, H, d, out=o, lse=lse)
        if a.kernel == "attn_fwd":
            ref = A.attn_reference(qkv[:2 * N], 2, N, H, d)
            out["rel_err_vs_fp32"] = ((o[:2 * N].float() - ref).norm() / ref.norm()).item()
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
    elif a.kernel == "modnorm_bwd":
        x = torch.randn(a.rows, a.dim, device=dev).bfloat16()
        dh, dres = torch.randn_like(x), torch.randn_like(x)
        sc, sh = torch.randn(a.dim, device=dev), torch.randn(a.dim, device=dev)
        w = torch.ones(a.dim, device=dev).bfloat16()
        dx = torch.empty_like(x)
        acc = [torch.zeros(a.dim, device=dev) for _ in range(3)]
        ms = _time(lambda: E.modnorm_bwd(x, dh, dres, sc, sh, w, mode=0, eps=1e-3, dx=dx, dscale=acc[0],
                                         dshift=acc[1], dw=acc[2]), a.iters)
        by = 4.0 * x.numel() * 2
        out.update(shape=[a.rows, a.dim], ms=ms, gbs=by / ms / 1e6, frac_of_peak=by / ms / 1e6 / bw_peak,
                   peak_source=src)
    elif a.kernel in ("embed", "loss"):
        from ..models import layout as LY
        from . import diffusion as DF
        grid = LY.Grid(720, 1440, 30, 30)
        geom = DF.make_geom(grid, 1, 0)
        x = torch.randn(1, 720, 1440, 70, device=dev)
        cs = torch.tensor([[0.6, 0.8]], device=dev)
        if a.kernel == "embed":
            c = torch.randn(1, 720, 1440, 74, device=dev)
            ay, ax = torch.randn(720, 72, device=dev), torch.randn(1440, 72, device=dev)
            A_ = torch.empty(geom.rows, 512, device=dev, dtype=torch.bfloat16)
            ms = _time(lambda: DF.embed_pack(x, c, cs, geom, ay, ax, 1, 1.0, True, A_), a.iters)
            by = geom.rows * (144 * 4 + 512 * 2.0)
        else:
            pred = torch.randn(geom.rows, 128, device=dev)
            dpred = torch.empty(geom.rows, 128, device=dev, dtype=torch.bfloat16)
            loss = torch.zeros(1, device=dev, dtype=torch.float64)
            wv, wl = torch.rand(70, device=dev), torch.rand(720, device=dev)
            ms = _time(lambda: DF.trigflow_loss(pred, x, cs, geom, 1, 1.0, wv, wl, 1.0 / geom.rows, loss, dpred=dpred),
                       a.iters)
            by = geom.rows * (128 * 4 + 70 * 4 + 128 * 2.0)
        out.update(rows=geom.rows, ms=ms, gbs=by / ms / 1e6, frac_of_peak=by / ms / 1e6 / bw_peak, peak_source=src)
    elif a.kernel.startswith("fused_"):
        import ctypes
        lib = L.lib()
        arr = lambda ts: (ctypes.c_void_p * len(ts))(*[t.data_ptr() for t in ts])
        st, sp_ = L.ptr(L.status_word()), L.stream_ptr
        if a.kernel == "fused_ag_gemm":
            M, K, N = a.m // 2 * 2, a.k, a.n
            bufs = [torch.randn(M, K, device=dev).bfloat16() for _ in range(2)]
            w = torch.randn(N, K, device=dev).bfloat16()
            c = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
            # rank 0's view: its own counters and a second array standing in for rank 1's; the chunk "pushed by rank 1"
            # is pre-filled and its arrival word pre-set, so the wait path runs and returns at once
            cnts = [torch.zeros(8, device=dev, dtype=torch.int32) for _ in range(2)]
            cnts[0][1] = 1 << 30
            full = bufs[0].clone()
            calls = [0]

            def run():
                calls[0] += 1
                L.check(lib.aeris_gemm_allgather_a(L.ptr(bufs[0]), arr(bufs), arr(cnts), 2, 0, M // 2,
                                                   ctypes.c_uint(calls[0]), L.ptr(w), L.ptr(c), N, K, K, N, 0, 0, None,
                                                   0, None, 0, 0, st, sp_()), "ag")
            run()
            ref = G.gemm(full, w)
            out["max_abs_diff_vs_plain_gemm"] = (c.float() - ref.float()).abs().max().item()
            ms = _time(run, a.iters)
            out.update(shape=[M, N, K], ms=ms, tflops=2.0 * M * N * K / ms / 1e9,
                       frac_of_peak=2.0 * M * N * K / ms / 1e9 / tf_peak, peak_source=src)
        elif a.kernel == "fused_rs_gemm":
            M, K, N = a.m // 2 * 2, a.k, a.n
            x = torch.randn(M, K, device=dev).bfloat16()
            w = torch.randn(N, K, device=dev).bfloat16()
            slots = [torch.zeros(M, N, device=dev, dtype=torch.bfloat16) for _ in range(2)]
            run = lambda: L.check(lib.aeris_gemm_rs_push(L.ptr(x), L.ptr(w), M, N, K, K, K, 0, arr(slots), 2, 0, M // 2, N,
                                                         st, sp_()), "rs")
            run()
            ref = G.gemm(x, w)
            got = torch.cat([slots[0][:M // 2], slots[1][:M // 2]])
            out["max_abs_diff_vs_plain_gemm"] = (got.float() - ref.float()).abs().max().item()
            ms = _time(run, a.iters)
            out.update(shape=[M, N, K], ms=ms, tflops=2.0 * M * N * K / ms / 1e9,
                       frac_of_peak=2.0 * M * N * K / ms / 1e9 / tf_peak, peak_source=src)
        elif a.kernel == "fused_scatter_heads":
            nw, L_, n_loc, H, d, K = a.windows, a.tokens, a.tokens // 2, a.heads, a.head_dim, a.dim
            HD = H * d
            x = torch.randn(nw * n_loc, K, device=dev).bfloat16()
            w = torch.randn(3 * HD, K, device=dev).bfloat16()
            dst = [torch.zeros(nw * L_, 3 * HD // 2, device=dev, dtype=torch.bfloat16) for _ in range(2)]
            run = lambda: L.check(lib.aeris_gemm_scatter_heads(L.ptr(x), L.ptr(w), nw * n_loc, 3 * HD, K, K, K, 0, arr(dst),
                                                               2, 0, n_loc, L_, HD, st, sp_()), "scatter")
            ms = _time(run, a.iters)
            fl = 2.0 * nw * n_loc * 3 * HD * K
            out.update(shape=[nw * n_loc, 3 * HD, K], ms=ms, tflops=fl / ms / 1e9, frac_of_peak=fl / ms / 1e9 / tf_peak,
                       peak_source=src)
        elif a.kernel in ("fused_grad_rs", "fused_shard_adamw"):
            n = a.rows * a.dim // 16 * 16
            per = n // 2
            if a.kernel == "fused_grad_rs":
                grads = [torch.randn(n, device=dev) for _ in range(2)]
                o = torch.empty(per, device=dev)
                ssq = torch.zeros(1, device=dev, dtype=torch.float64)
                run = lambda: L.check(lib.aeris_grad_reduce_scatter(arr(grads), None, 2, L._c_ll(0), L._c_ll(per),
                                                                    L._c_float(0.5), L.ptr(o), L.ptr(ssq), sp_()), "rs")
                by = per * 4 * 3.0
            else:
                params = [torch.empty(n, device=dev, dtype=torch.bfloat16) for _ in range(2)]
                b5 = [torch.randn(per, device=dev) for _ in range(5)]
                b5[3].abs_()
                f = L._c_float
                run = lambda: L.check(lib.aeris_shard_adamw_allgather(
                    L.ptr(b5[0]), L.ptr(b5[1]), L.ptr(b5[2]), L.ptr(b5[3]), L.ptr(b5[4]), arr(params), None, 2,
                    L._c_ll(0), L._c_ll(per), None, f(1e-4), f(0.9), f(0.99), f(1e-8), f(0.0), 3, f(0.0), f(0.999),
                    sp_()), "adamw")
                by = per * (5 * 4 + 4 * 4 + 2 * 2.0)
            ms = _time(run, a.iters)
            out.update(n=per, ms=ms, gbs=by / ms / 1e6, frac_of_peak=by / ms / 1e6 / bw_peak, peak_source=src)
        else:
            from ..models import layout as LY
            grid = LY.Grid(720, 1440, 30, 30, 1, 2)
            rows, D = grid.tokens_per_rank, a.dim
            table = LY.gather_table(grid, (0, 0), grid.half_shift(), 0).to(dev)
            xs = [torch.randn(rows, D, device=dev).bfloat16() for _ in range(2)]
            sc, sh = torch.randn(D, device=dev), torch.randn(D, device=dev)
            w = torch.ones(D, device=dev).bfloat16()
            h, xg = torch.empty_like(xs[0]), torch.empty_like(xs[0])
            ms = _time(lambda: E.modnorm_fwd(None, sc, sh, w, mode=0, eps=1e-3, out=h, gather_idx=table,
                                             peer_ptrs=[t.data_ptr() for t in xs], x_out=xg, rows=rows), a.iters)
            by = rows * D * 2 * 3.0
            out.update(shape=[rows, D], ms=ms, gbs=by / ms / 1e6, frac_of_peak=by / ms / 1e6 / bw_peak, peak_source=src)
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
    out["clocks"] = _CLOCKS[-1] if _CLOCKS else None
    print(json.dumps(out))


if __name__ == "__main__":
    main()
