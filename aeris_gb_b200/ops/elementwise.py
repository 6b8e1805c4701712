"""Python front ends of the memory-bound kernels in ``csrc/elementwise.cu``."""
from __future__ import annotations

import ctypes

import torch

from . import lib as _l
from .build import CHECKED as _CHECKED

MODE_MOD_THEN_NORM = 0   # h = RMSNorm(x * (1 + scale) + shift) * w      (layerwise_t_emb_after_mod_norm)
MODE_NORM_THEN_MOD = 1   # h = (RMSNorm(x) * w) * (1 + scale) + shift    (DiT ordering)


def _peer_array(ptrs: list[int]):
    arr = (ctypes.c_void_p * len(ptrs))(*ptrs)
    return arr


def modnorm_fwd(x: torch.Tensor, scale: torch.Tensor | None, shift: torch.Tensor | None, w: torch.Tensor, *,
                mode: int, eps: float, out: torch.Tensor | None = None, gather_idx: torch.Tensor | None = None,
                peer_ptrs: list[int] | None = None, x_out: torch.Tensor | None = None,
                rows: int | None = None, out_lo: torch.Tensor | None = None,
                src_rows: int | None = None) -> torch.Tensor:
    """``w`` bf16, or fp32 (the output head's norm); ``out_lo`` optionally receives ``h - bf16(h)``. ``src_rows``:
    rows of every peer buffer the gather table points into (used by the checking build only)."""
    D = w.numel()
    rows = rows if rows is not None else (gather_idx.numel() if gather_idx is not None else x.shape[0])
    if _CHECKED and gather_idx is not None:
        set_gather_bounds(src_rows or 0)
    if out is None:
        out = torch.empty((rows, D), dtype=torch.bfloat16, device=w.device)
    peers = _peer_array(peer_ptrs) if gather_idx is not None else None
    w32, w = (w, None) if w.dtype == torch.float32 else (None, w)
    rc = _l.lib().aeris_modnorm_fwd(_l.ptr(x), _l.ptr(gather_idx), peers, len(peer_ptrs) if peer_ptrs else 0,
                                    _l.ptr(x_out), _l.ptr(scale), _l.ptr(shift), _l.ptr(w), _l.ptr(out), rows, D,
                                    mode, _l._c_float(eps), _l.ptr(w32), _l.ptr(out_lo), _l.stream_ptr())
    _l.check(rc, "aeris_modnorm_fwd")
    return out


def modnorm_bwd(x: torch.Tensor, dh: torch.Tensor, dres: torch.Tensor | None, scale: torch.Tensor | None,
                shift: torch.Tensor | None, w: torch.Tensor, *, mode: int, eps: float, dx: torch.Tensor,
                dscale: torch.Tensor | None, dshift: torch.Tensor | None, dw: torch.Tensor | None) -> torch.Tensor:
    rows, D = x.shape
    w32, w = (w, None) if w.dtype == torch.float32 else (None, w)
    rc = _l.lib().aeris_modnorm_bwd(_l.ptr(x), _l.ptr(dh), _l.ptr(dres), _l.ptr(scale), _l.ptr(shift), _l.ptr(w),
                                    _l.ptr(dx), _l.ptr(dscale), _l.ptr(dshift), _l.ptr(dw), rows, D, mode,
                                    _l._c_float(eps), _l.ptr(w32), _l.stream_ptr())
    _l.check(rc, "aeris_modnorm_bwd")
    return dx


def set_gather_bounds(src_rows: int) -> bool:
    """Checking build (AERIS_BOUNDS_CHECK=1) only: rows of the source buffers of the gathers launched next, so that
    every table entry is validated on the device. Returns whether the loaded library checks at all."""
    return bool(_l.lib().aeris_debug_set_gather_bounds(_l.ptr(_l.status_word()), int(src_rows)))


def gather_rows(gather_idx: torch.Tensor, peer_ptrs: list[int], out: torch.Tensor,
                src_rows: int | None = None) -> torch.Tensor:
    rows, D = out.shape
    if _CHECKED:
        set_gather_bounds(src_rows or 0)
    rc = _l.lib().aeris_gather_rows(_l.ptr(gather_idx), _peer_array(peer_ptrs), len(peer_ptrs), _l.ptr(out),
                                    _l._c_ll(rows), D, _l.stream_ptr())
    _l.check(rc, "aeris_gather_rows")
    return out


def swiglu_fwd(u: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    rows, F2 = u.shape
    F = F2 // 2
    if out is None:
        out = torch.empty((rows, F), dtype=u.dtype, device=u.device)
    _l.check(_l.lib().aeris_swiglu_fwd(_l.ptr(u), _l.ptr(out), _l._c_ll(rows), F, _l.stream_ptr()), "swiglu_fwd")
    return out


def swiglu_bwd(u: torch.Tensor, dact: torch.Tensor, du: torch.Tensor | None = None) -> torch.Tensor:
    rows, F2 = u.shape
    if du is None:
        du = torch.empty_like(u)
    _l.check(_l.lib().aeris_swiglu_bwd(_l.ptr(u), _l.ptr(dact), _l.ptr(du), _l._c_ll(rows), F2 // 2,
                                       _l.stream_ptr()), "swiglu_bwd")
    return du


def scale_rows(W: torch.Tensor, g: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    R, C = W.shape
    if out is None:
        out = torch.empty_like(W)
    _l.check(_l.lib().aeris_scale_rows(_l.ptr(W), _l.ptr(g), _l.ptr(out), R, C, _l.stream_ptr()), "scale_rows")
    return out


def rope_qk_(qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, L: int, heads: int, head_dim: int,
             inverse: bool = False) -> torch.Tensor:
    """Rotates the q and k sections of ``qkv`` [rows, 3 * heads * head_dim] (bf16, contiguous) in place by the 2-D rotary
    angles ``cos`` / ``sin`` [L, head_dim / 2] (fp32); row r belongs to token r mod L of its window."""
    assert qkv.is_contiguous() and qkv.shape[1] == 3 * heads * head_dim and cos.shape == (L, head_dim // 2)
    _l.check(_l.lib().aeris_rope_qk(_l.ptr(qkv), _l.ptr(cos), _l.ptr(sin), _l._c_ll(qkv.shape[0]), L, heads, head_dim,
                                    int(inverse), _l.stream_ptr()), "rope_qk")
    return qkv


def gate_grad_finalize(G: torch.Tensor, W: torch.Tensor, g: torch.Tensor, dW: torch.Tensor, dg: torch.Tensor) -> None:
    R, C = W.shape
    _l.check(_l.lib().aeris_gate_grad_finalize(_l.ptr(G), _l.ptr(W), _l.ptr(g), _l.ptr(dW), _l.ptr(dg), R, C,
                                               _l.stream_ptr()), "gate_grad_finalize")


def sumsq(x: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    _l.check(_l.lib().aeris_sumsq(_l.ptr(x), _l._c_ll(x.numel()), _l.ptr(out), _l.stream_ptr()), "sumsq")
    return out


def adamw(master: torch.Tensor, grad: torch.Tensor, m: torch.Tensor, v: torch.Tensor, wbf16: torch.Tensor | None,
          ema: torch.Tensor | None, norm_sq: torch.Tensor | None, *, lr: float, betas: tuple[float, float],
          eps: float, weight_decay: float, step: int, grad_scale: float, max_norm: float, ema_beta: float) -> None:
    f = _l._c_float
    _l.check(_l.lib().aeris_adamw(_l.ptr(master), _l.ptr(grad), _l.ptr(m), _l.ptr(v), _l.ptr(wbf16), _l.ptr(ema),
                                  _l.ptr(norm_sq), _l._c_ll(master.numel()), f(lr), f(betas[0]), f(betas[1]),
                                  f(eps), f(weight_decay), step, f(grad_scale), f(max_norm), f(ema_beta),
                                  _l.stream_ptr()), "adamw")
