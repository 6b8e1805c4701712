"""CUDA execution of the two ends of the network: noising + position encoding + input projection, and the fp32 output
head with the TrigFlow loss.

Both ends are fp32 in the reference (src/aeris/models/parallel_swin.py:383-386 and :519-529, the loss at
src/aeris/parallelism/parallel_engine.py:990-997). Here their contractions run on the bf16 tensor cores at fp32-level
accuracy by splitting each fp32 operand into a bf16 value and a bf16 remainder and summing the three significant
products (hi*hi + lo*hi + hi*lo); the rest (noise, mixing, position encoding, window partition, norm, modulation,
loss and its gradient) lives in the element-wise kernels around them, so the fp32 model input, the noise and the
prediction error never exist in memory as full-size tensors.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..ops import diffusion as DF
from ..ops import elementwise as E
from ..ops import gemm as G
from . import oracle as O
from .fused import workspace

PAD_N = 128          # output channels are padded to one GEMM tile
CHUNK_ROWS = 1 << 16


@dataclass
class IoPlan:
    """What the fused input/output ends need to know about one training or sampling call."""
    geom: DF.TokGeom
    sigma_data: float
    seed: int = 0
    noise: bool = True
    ape_y: torch.Tensor | None = None     # [H (+offset applied), ch] fp32
    ape_x: torch.Tensor | None = None     # [W, ch] fp32
    w_var: torch.Tensor | None = None     # [C_out] fp32
    w_lat: torch.Tensor | None = None     # [H] fp32 (global image rows)
    eps: float = 1.1920929e-07


def ape_tables(cfg, device) -> tuple[torch.Tensor, torch.Tensor]:
    off = cfg.ape_row_offset if cfg.ape_row_offset is not None else (1 if cfg.img[0] == 720 else 0)
    ty, tx = O.positional_tables(cfg.in_channels, cfg.img[0] + off, cfg.img[1])
    return ty[off:].contiguous().to(device), tx.contiguous().to(device)


def _split(t: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    hi = t.to(torch.bfloat16)
    return hi, (t - hi.float()).to(torch.bfloat16)


def _grad_slot(p: torch.Tensor):
    """fp32 accumulation target of a parameter: the engine's ``main_grad`` view, or a fresh buffer handed back to
    autograd."""
    mg = getattr(p, "main_grad", None)
    if mg is not None:
        return (mg.view(p.shape) if mg.shape != p.shape else mg), None
    z = torch.zeros(p.shape, dtype=torch.float32, device=p.device)
    return z, z


def _pack_dim(c_in: int) -> int:
    return (3 * c_in + 2 + 127) // 128 * 128


class EmbedFn(torch.autograd.Function):
    """``(cat[(cos t x + sin t z) / sigma_d, cond] + ape) W^T + b`` -> bf16 token stream in the unshifted window layout."""

    @staticmethod
    def forward(ctx, x_img, c_img, cs, W, b, plan: IoPlan):
        D, Cin = W.shape
        KP = _pack_dim(Cin)
        dev = x_img.device
        Wp = torch.zeros((D, KP), dtype=torch.bfloat16, device=dev)
        w_hi, w_lo = _split(W.detach().float())
        b_hi, b_lo = _split(b.detach().float())
        Wp[:, :Cin], Wp[:, Cin:2 * Cin], Wp[:, 2 * Cin:3 * Cin] = w_hi, w_hi, w_lo
        Wp[:, 3 * Cin], Wp[:, 3 * Cin + 1] = b_hi, b_lo
        T = plan.geom.rows
        out = torch.empty((T, D), dtype=torch.bfloat16, device=dev)
        A = workspace().get("embed_a", (min(CHUNK_ROWS, T), KP), torch.bfloat16, dev)
        for r0 in range(0, T, CHUNK_ROWS):
            n = min(CHUNK_ROWS, T - r0)
            DF.embed_pack(x_img, c_img, cs, plan.geom, plan.ape_y, plan.ape_x, plan.seed, plan.sigma_data,
                          plan.noise, A[:n], row0=r0)
            G.gemm(A[:n], Wp, out=out[r0:r0 + n])
        ctx.plan = plan
        ctx.save_for_backward(x_img, c_img, cs, W, b)
        return out

    @staticmethod
    def backward(ctx, dout):
        x_img, c_img, cs, W, b = ctx.saved_tensors
        plan = ctx.plan
        D, Cin = W.shape
        KP = _pack_dim(Cin)
        dev = dout.device
        dout = dout.contiguous()
        T = plan.geom.rows
        A = workspace().get("embed_a", (min(CHUNK_ROWS, T), KP), torch.bfloat16, dev)
        Gw = workspace().get("embed_g", (D, KP), torch.float32, dev, zero=True)
        for r0 in range(0, T, CHUNK_ROWS):
            n = min(CHUNK_ROWS, T - r0)
            DF.embed_pack(x_img, c_img, cs, plan.geom, plan.ape_y, plan.ape_x, plan.seed, plan.sigma_data,
                          plan.noise, A[:n], row0=r0)
            G.gemm(dout[r0:r0 + n], A[:n], a_t=True, b_t=True, out=Gw, epi=G.EPI_ACC_F32, k_splits=8)
        dW = Gw[:, :Cin] + Gw[:, Cin:2 * Cin]
        db = Gw[:, 3 * Cin]
        sW, rW = _grad_slot(W)
        sb, rb = _grad_slot(b)
        sW += dW
        sb += db
        return (None, None, None, rW.to(W.dtype) if rW is not None else None,
                rb.to(b.dtype) if rb is not None else None, None)


def _head_weights(head_w: torch.Tensor):
    C, D = head_w.shape
    hi, lo = _split(head_w.detach().float())
    w_hi = torch.zeros((PAD_N, D), dtype=torch.bfloat16, device=head_w.device)
    w_lo = torch.zeros((PAD_N, D), dtype=torch.bfloat16, device=head_w.device)
    w_hi[:C], w_lo[:C] = hi, lo
    return w_hi, w_lo


def _head_rows(x, scale_b, shift_b, norm_w, w_hi, w_lo, eps, pred, y_hi, y_lo):
    """pred[n, 128] (fp32) = (RMSNorm(x) * w * (1 + scale) + shift) @ head^T for ``n`` rows of one sample."""
    n = x.shape[0]
    E.modnorm_fwd(x, scale_b, shift_b, norm_w, mode=E.MODE_NORM_THEN_MOD, eps=eps, out=y_hi[:n], out_lo=y_lo[:n])
    G.gemm(y_hi[:n], w_hi, out=pred[:n], epi=G.EPI_STORE_F32)
    G.gemm(y_lo[:n], w_hi, out=pred[:n], epi=G.EPI_ACC_F32)
    G.gemm(y_hi[:n], w_lo, out=pred[:n], epi=G.EPI_ACC_F32)
    return pred[:n]


def _sample_chunks(B: int, rows_per_sample: int):
    for b in range(B):
        for r in range(0, rows_per_sample, CHUNK_ROWS):
            yield b, b * rows_per_sample + r, min(CHUNK_ROWS, rows_per_sample - r)


def head_forward(x: torch.Tensor, shift: torch.Tensor, scale: torch.Tensor, norm_w: torch.Tensor,
                 head_w: torch.Tensor, eps: float) -> torch.Tensor:
    """Network output ``F`` in token order, fp32 ``[T, 128]`` (columns past the channel count are zero)."""
    T, D = x.shape
    B = shift.shape[0]
    dev = x.device
    w_hi, w_lo = _head_weights(head_w)
    ws = workspace()
    cm = min(CHUNK_ROWS, T // B)
    y_hi = ws.get("head_yhi", (cm, D), torch.bfloat16, dev)
    y_lo = ws.get("head_ylo", (cm, D), torch.bfloat16, dev)
    pred = torch.empty((T, PAD_N), dtype=torch.float32, device=dev)
    shift, scale = shift.float().contiguous(), scale.float().contiguous()
    for b, r0, n in _sample_chunks(B, T // B):
        _head_rows(x[r0:r0 + n], scale[b], shift[b], norm_w, w_hi, w_lo, eps, pred[r0:r0 + n], y_hi, y_lo)
    return pred


class HeadLossFn(torch.autograd.Function):
    """Output head + TrigFlow loss: returns ``sum_b mean_rows sum_c w_lat w_var (sigma_d F - v_t)^2`` as a scalar.
    Forward keeps the stream input and d loss / d F (bf16, 128 columns per row); backward recomputes the normalised
    rows chunk by chunk."""

    @staticmethod
    def forward(ctx, x, shift, scale, norm_w, head_w, x_img, cs, plan: IoPlan):
        T, D = x.shape
        B = shift.shape[0]
        dev = x.device
        w_hi, w_lo = _head_weights(head_w)
        ws = workspace()
        cm = min(CHUNK_ROWS, T // B)
        y_hi = ws.get("head_yhi", (cm, D), torch.bfloat16, dev)
        y_lo = ws.get("head_ylo", (cm, D), torch.bfloat16, dev)
        pred = ws.get("head_pred", (cm, PAD_N), torch.float32, dev)
        dpred = torch.empty((T, PAD_N), dtype=torch.bfloat16, device=dev)
        loss = torch.zeros(1, dtype=torch.float64, device=dev)
        shift32, scale32 = shift.float().contiguous(), scale.float().contiguous()
        inv_rows = 1.0 / (T // B)
        for b, r0, n in _sample_chunks(B, T // B):
            _head_rows(x[r0:r0 + n], scale32[b], shift32[b], norm_w, w_hi, w_lo, plan.eps, pred, y_hi, y_lo)
            DF.trigflow_loss(pred[:n], x_img, cs, plan.geom, plan.seed, plan.sigma_data, plan.w_var, plan.w_lat,
                             inv_rows, loss, dpred=dpred[r0:r0 + n], row0=r0)
        ctx.plan = plan
        ctx.save_for_backward(x, shift, scale, norm_w, head_w, dpred)
        return loss.float().squeeze(0)

    @staticmethod
    def backward(ctx, g):
        x, shift, scale, norm_w, head_w, dpred = ctx.saved_tensors
        plan = ctx.plan
        T, D = x.shape
        B = shift.shape[0]
        C = head_w.shape[0]
        dev = x.device
        w_hi, _ = _head_weights(head_w)
        ws = workspace()
        cm = min(CHUNK_ROWS, T // B)
        y_hi = ws.get("head_yhi", (cm, D), torch.bfloat16, dev)
        dy = ws.get("head_ylo", (cm, D), torch.bfloat16, dev)
        Gh = ws.get("head_g", (PAD_N, D), torch.float32, dev, zero=True)
        shift32, scale32 = shift.float().contiguous(), scale.float().contiguous()
        dshift, dscale = torch.zeros_like(shift32), torch.zeros_like(scale32)
        s_nw, r_nw = _grad_slot(norm_w)
        dnw = torch.zeros(D, dtype=torch.float32, device=dev)
        dx = torch.empty_like(x)
        dpred = dpred * g.to(dpred.dtype)
        for b, r0, n in _sample_chunks(B, T // B):
            E.modnorm_fwd(x[r0:r0 + n], scale32[b], shift32[b], norm_w, mode=E.MODE_NORM_THEN_MOD, eps=plan.eps,
                          out=y_hi[:n])
            dp = dpred[r0:r0 + n]
            G.gemm(dp, y_hi[:n], a_t=True, b_t=True, out=Gh, epi=G.EPI_ACC_F32, k_splits=16, two_cta=False)
            G.gemm(dp, w_hi, b_t=True, out=dy[:n])
            E.modnorm_bwd(x[r0:r0 + n], dy[:n], None, scale32[b], shift32[b], norm_w, mode=E.MODE_NORM_THEN_MOD,
                          eps=plan.eps, dx=dx[r0:r0 + n], dscale=dscale[b], dshift=dshift[b], dw=dnw)
        s_nw += dnw
        s_hw, r_hw = _grad_slot(head_w)
        s_hw += Gh[:C]
        return (dx, dshift.to(shift.dtype), dscale.to(scale.dtype), r_nw.to(norm_w.dtype) if r_nw is not None else None,
                r_hw.to(head_w.dtype) if r_hw is not None else None, None, None, None)
