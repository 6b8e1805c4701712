"""SWiPe layouts: how the tokens of one sample are spread over (window-parallel rank, sequence-parallel rank) at each
pipeline stage, and the routes that move them between consecutive stages.

Reference scheme (src/aeris/parallelism/parallel_engine.py:175-199, 335-373, 462-583, 933-954):
  * windows are dealt round-robin to the WP grid: window (wy, wx) -> WP rank (wy mod WP_Y, wx mod WP_X);
  * every window is cut into four quadrants (TL, TR, BL, BR), each quadrant into SP/4 contiguous chunks;
    SP rank = quadrant * (SP/4) + chunk (SP is hard-wired to 12 there);
  * the half-window shift costs no extra communication: the pipeline send between stages delivers each chunk to the
    rank that owns it in the *shifted* window grid (TL -> BR of the WP neighbour up-left, TR -> BL of the neighbour
    above, BL -> TR of the left neighbour, BR -> TL in place), plus a roll of the local window index on wrap-around
    ranks; the next transition undoes it.

Here the scheme is stated once, generically: a *layout* maps every pixel to (wp_y, wp_x, sp, row); the route between
two layouts is derived from the two maps, for any SP in {1, 2, 4k}, any WP grid and any even window. The reference's
hand-written tables are the special case SP = 12; the tests check that.
"""
from __future__ import annotations

from dataclasses import dataclass
from functools import lru_cache

import numpy as np


@dataclass(frozen=True)
class SwipeGeometry:
    H: int
    W: int
    ws_y: int
    ws_x: int
    WP_Y: int
    WP_X: int
    SP: int

    def __post_init__(self):
        assert self.ws_y % 2 == 0 and self.ws_x % 2 == 0, "windows must split into equal halves"
        assert self.H % self.ws_y == 0 and self.W % self.ws_x == 0
        assert (self.H // self.ws_y) % self.WP_Y == 0 and (self.W // self.ws_x) % self.WP_X == 0
        assert self.SP in (1, 2) or self.SP % 4 == 0, "SP must be 1, 2 or a multiple of 4 (quadrant x chunk split)"
        q = (self.ws_y // 2) * (self.ws_x // 2)
        if self.SP >= 4:
            assert q % (self.SP // 4) == 0, "a quadrant must split evenly into SP/4 chunks"

    @property
    def nwy(self):
        return self.H // self.ws_y

    @property
    def nwx(self):
        return self.W // self.ws_x

    @property
    def local_windows(self):
        return (self.nwy // self.WP_Y) * (self.nwx // self.WP_X)

    @property
    def tokens_per_sp_rank(self):
        return self.ws_y * self.ws_x // self.SP


@lru_cache(maxsize=32)
def ownership(g: SwipeGeometry, shifted: bool):
    """For every pixel: (wp_y, wp_x, sp, row) in the plain (shifted=False) or half-window-shifted layout.

    Row order inside an SP rank is (local window index, token within the chunk); a window's tokens are ordered
    quadrant-major (TL, TR, BL, BR), row-major inside a quadrant, and the SP rank takes a contiguous slice: with
    SP >= 4 a chunk of one quadrant, with SP = 2 the top or bottom pair of quadrants, with SP = 1 everything.
    """
    hy, hx = g.ws_y // 2, g.ws_x // 2
    sy, sx = (hy, hx) if shifted else (0, 0)
    y = (np.arange(g.H) - sy) % g.H
    x = (np.arange(g.W) - sx) % g.W
    wy, iy = (y // g.ws_y)[:, None], (y % g.ws_y)[:, None]
    wx, ix = (x // g.ws_x)[None, :], (x % g.ws_x)[None, :]
    wp_y, ly = wy % g.WP_Y, wy // g.WP_Y
    wp_x, lx = wx % g.WP_X, wx // g.WP_X
    quad = (iy // hy) * 2 + (ix // hx)
    in_q = (iy % hy) * hx + (ix % hx)
    seq = quad * (hy * hx) + in_q                       # position in the quadrant-major window sequence
    per = g.tokens_per_sp_rank
    sp = seq // per
    tok = seq % per
    lw = ly * (g.nwx // g.WP_X) + lx
    row = lw * per + tok
    shape = (g.H, g.W)
    return (np.broadcast_to(wp_y, shape).copy(), np.broadcast_to(wp_x, shape).copy(),
            np.broadcast_to(sp, shape).copy(), np.broadcast_to(row, shape).copy())


def route(g: SwipeGeometry, src_shifted: bool, dst_shifted: bool, wp_y: int, wp_x: int, sp: int):
    """Rows this (wp_y, wp_x, sp) coordinate must SEND when moving from the src to the dst layout.

    Returns ``{(dst_wp_y, dst_wp_x, dst_sp): (src_rows, dst_rows)}`` with matching int64 arrays sorted by dst row."""
    sy_, sx_, ss_, sr_ = ownership(g, src_shifted)
    dy_, dx_, ds_, dr_ = ownership(g, dst_shifted)
    mine = (sy_ == wp_y) & (sx_ == wp_x) & (ss_ == sp)
    out = {}
    keys = np.stack([dy_[mine], dx_[mine], ds_[mine]], axis=1)
    srow, drow = sr_[mine], dr_[mine]
    for key in np.unique(keys, axis=0):
        sel = (keys == key).all(axis=1)
        order = np.argsort(drow[sel], kind="stable")
        out[tuple(int(k) for k in key)] = (srow[sel][order], drow[sel][order])
    return out


def recv_plan(g: SwipeGeometry, src_shifted: bool, dst_shifted: bool, wp_y: int, wp_x: int, sp: int):
    """Mirror of :func:`route`: ``{(src coords): (src_rows, dst_rows)}`` for the rows this coordinate RECEIVES."""
    sy_, sx_, ss_, sr_ = ownership(g, src_shifted)
    dy_, dx_, ds_, dr_ = ownership(g, dst_shifted)
    mine = (dy_ == wp_y) & (dx_ == wp_x) & (ds_ == sp)
    out = {}
    keys = np.stack([sy_[mine], sx_[mine], ss_[mine]], axis=1)
    srow, drow = sr_[mine], dr_[mine]
    for key in np.unique(keys, axis=0):
        sel = (keys == key).all(axis=1)
        order = np.argsort(drow[sel], kind="stable")
        out[tuple(int(k) for k in key)] = (srow[sel][order], drow[sel][order])
    return out


def stage_is_shifted(pp_rank: int, n_stages: int) -> bool:
    """Middle stages alternate, starting unshifted at stage 1; the first and last stage use the plain layout
    (reference: ``shift_up_next = pp_rank % 2 == 1`` with stage 0 -> 1 never shifting, :314, :365-373)."""
    if pp_rank == 0 or pp_rank == n_stages - 1:
        return False
    return pp_rank % 2 == 0


def reference_next_rank_sp12(wp_y: int, wp_x: int, sp: int, WP_Y: int, WP_X: int, shift_up_next: bool):
    """The reference's hand-written SP = 12 routing table (:335-364), kept as a test oracle for :func:`route`."""
    if shift_up_next:
        table = [(-1, -1, +9), (-1, 0, +3), (0, -1, -3), (0, 0, -9)]
    else:
        table = [(0, 0, +9), (0, +1, +3), (+1, 0, -3), (+1, +1, -9)]
    dy, dx, dsp = table[sp // 3]
    return (wp_y + dy) % WP_Y, (wp_x + dx) % WP_X, sp + dsp


def tile_sample(img: np.ndarray, g: SwipeGeometry, shifted: bool, wp_y: int, wp_x: int, sp: int) -> np.ndarray:
    """``img [H, W, C]`` -> the rows ``[local_windows * tokens_per_sp_rank, C]`` one coordinate holds."""
    oy, ox, os_, orow = ownership(g, shifted)
    mine = (oy == wp_y) & (ox == wp_x) & (os_ == sp)
    ys, xs = np.nonzero(mine)
    order = np.argsort(orow[ys, xs], kind="stable")
    return img[ys[order], xs[order]]
