"""Python front ends of ``csrc/diffusion.cu``: noising + embedding pack, TrigFlow loss, sampler updates, channel
affine maps and the small-batch GEMV of the modulation MLPs."""
from __future__ import annotations

import ctypes

import torch

from . import lib as _l


class TokGeom(ctypes.Structure):
    """Mirror of the C struct: this rank's token stream / image block inside the global image."""
    _fields_ = [("B", ctypes.c_int), ("nwy_loc", ctypes.c_int), ("nwx_loc", ctypes.c_int), ("ws_y", ctypes.c_int),
                ("ws_x", ctypes.c_int), ("n_local", ctypes.c_int), ("sp_rank", ctypes.c_int), ("y0", ctypes.c_int),
                ("x0", ctypes.c_int), ("H", ctypes.c_int), ("W", ctypes.c_int), ("sample0", ctypes.c_longlong)]

    @property
    def rows(self) -> int:
        return self.B * self.nwy_loc * self.nwx_loc * self.n_local

    @property
    def block_shape(self) -> tuple[int, int, int]:
        return self.B, self.nwy_loc * self.ws_y, self.nwx_loc * self.ws_x


def make_geom(grid, batch: int, rank: int = 0, sample0: int = 0) -> TokGeom:
    """Geometry of ``rank`` (= wp_rank * sp + sp_rank) of a :class:`aeris_gb_b200.models.layout.Grid`."""
    ry, rx = grid.rank_coords(rank)
    return TokGeom(batch, grid.nwy_loc, grid.nwx_loc, grid.ws_y, grid.ws_x, grid.n_local, rank % grid.sp,
                   ry * grid.nwy_loc * grid.ws_y, rx * grid.nwx_loc * grid.ws_x, grid.H, grid.W, sample0)


def _u64(v: int) -> ctypes.c_ulonglong:
    return ctypes.c_ulonglong(v & 0xFFFFFFFFFFFFFFFF)


def embed_pack(x_img: torch.Tensor, c_img: torch.Tensor | None, cs: torch.Tensor, g: TokGeom,
               ape_y: torch.Tensor | None, ape_x: torch.Tensor | None, seed: int, sigma_data: float, noise: bool,
               out: torch.Tensor, row0: int = 0) -> torch.Tensor:
    """Rows ``[row0, row0 + out.shape[0])`` of the packed model input ``[hi | lo | hi | 1 | 1 | 0..]`` (bf16)."""
    Cx = x_img.shape[-1]
    Cc = c_img.shape[-1] if c_img is not None else 0
    rc = _l.lib().aeris_embed_pack(_l.ptr(x_img), _l.ptr(c_img), _l.ptr(cs), ctypes.byref(g), Cx, Cc, _l.ptr(ape_y),
                                   _l.ptr(ape_x), ape_y.shape[1] if ape_y is not None else 0, _u64(seed),
                                   _l._c_float(sigma_data), int(noise), _l.ptr(out), out.stride(0),
                                   _l._c_ll(row0), _l._c_ll(out.shape[0]), _l.stream_ptr())
    _l.check(rc, "aeris_embed_pack")
    return out


def trigflow_loss(pred: torch.Tensor, x_img: torch.Tensor, cs: torch.Tensor, g: TokGeom, seed: int,
                  sigma_data: float, w_var: torch.Tensor | None, w_lat: torch.Tensor | None, inv_rows: float,
                  loss: torch.Tensor, dpred: torch.Tensor | None = None, gscale: float = 1.0, row0: int = 0) -> None:
    """Adds the loss of ``pred.shape[0]`` rows starting at ``row0`` to ``loss`` (float64 [1]); writes d loss / d pred."""
    rc = _l.lib().aeris_trigflow_loss(_l.ptr(pred), pred.stride(0), _l.ptr(x_img), _l.ptr(cs), ctypes.byref(g),
                                      x_img.shape[-1], _u64(seed), _l._c_float(sigma_data), _l.ptr(w_var),
                                      _l.ptr(w_lat), _l._c_float(inv_rows), _l._c_float(gscale), _l.ptr(dpred),
                                      dpred.stride(0) if dpred is not None else 4, _l.ptr(loss), _l._c_ll(row0),
                                      _l._c_ll(pred.shape[0]), _l.stream_ptr())
    _l.check(rc, "aeris_trigflow_loss")


def sampler_update(x_out: torch.Tensor, x_base: torch.Tensor, pa: torch.Tensor, pb: torch.Tensor | None, ca: float,
                   cb: float, g: TokGeom) -> torch.Tensor:
    """``x_out = x_base + ca * pa + cb * pb`` with ``pa, pb`` [rows, ld] fp32 in token order, x in image order."""
    rc = _l.lib().aeris_sampler_update(_l.ptr(x_out), _l.ptr(x_base), _l.ptr(pa), _l.ptr(pb), pa.stride(0),
                                       _l._c_float(ca), _l._c_float(cb), ctypes.byref(g), x_out.shape[-1],
                                       _l.stream_ptr())
    _l.check(rc, "aeris_sampler_update")
    return x_out


def noise_mix(x: torch.Tensor, a: float, b: float, seed: int, g: TokGeom) -> torch.Tensor:
    """In place ``x = a * x + b * z`` with z ~ N(0, 1) from the counter-based generator (x: [B, hb, wb, C] fp32)."""
    rc = _l.lib().aeris_noise_mix(_l.ptr(x), _l._c_float(a), _l._c_float(b), _u64(seed), ctypes.byref(g),
                                  x.shape[-1], _l.stream_ptr())
    _l.check(rc, "aeris_noise_mix")
    return x


def affine_channels(inp: torch.Tensor, a: torch.Tensor, b: torch.Tensor, add: torch.Tensor | None = None,
                    out: torch.Tensor | None = None) -> torch.Tensor:
    """``out = inp * a[c] + b[c] (+ add)`` over the last (channel) axis, fp32."""
    if out is None:
        out = torch.empty_like(inp)
    rc = _l.lib().aeris_affine_channels(_l.ptr(out), _l.ptr(inp), _l.ptr(a), _l.ptr(b), _l.ptr(add),
                                        _l._c_ll(inp.numel()), inp.shape[-1], _l.stream_ptr())
    _l.check(rc, "aeris_affine_channels")
    return out


def gemv_bias_act(W: torch.Tensor, bias: torch.Tensor | None, x: torch.Tensor, act: int = 0,
                  silu_in: bool = False) -> torch.Tensor:
    """``act(silu?(x) @ W^T + bias)`` for at most 8 rows of fp32 ``x``; W bf16 or fp32 [N, K]; fp32 result."""
    N, K = W.shape
    B = x.shape[0]
    y = torch.empty((B, N), dtype=torch.float32, device=x.device)
    rc = _l.lib().aeris_gemv_bias_act(_l.ptr(W), int(W.dtype == torch.float32), _l.ptr(bias), _l.ptr(x), _l.ptr(y), N,
                                      K, B, act, int(silu_in), _l.stream_ptr())
    _l.check(rc, "aeris_gemv_bias_act")
    return y
