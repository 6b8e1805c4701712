"""Window layouts of the token stream and the gather tables that move between them.

The residual stream is kept *window-major*: for a layer whose windows are offset by ``shift`` pixels (0 for plain
layers, ``window // 2`` for shifted layers; the shift is periodic in both axes and unmasked, as in the reference,
``src/aeris_wp_inference/model.py:49-60,111-114`` and ``src/aeris/parallelism/parallel_engine.py:335-373``), token
``((b * nWy + wy) * nWx + wx) * L + iy * ws_x + ix`` holds pixel ``((wy * ws_y + iy + shift_y) mod H,
(wx * ws_x + ix + shift_x) mod W)`` of sample ``b``.

With window parallelism (WP) a ``wp_y x wp_x`` grid of ranks each owns a contiguous block of *windows* of the
current layout (reference: contiguous blocks per rank, ``src/aeris_wp_inference/era5.py:249-277``). Moving from
the plain to the shifted layout therefore needs rows that live on up to three neighbour ranks: the halo exchange.
A *gather table* lists, for every destination row of this rank, ``(source rank << 28) | source row``; the CUDA
kernels read source rows straight from peer memory with it, so the exchange is fused into the consumer kernel.
"""
from __future__ import annotations

from dataclasses import dataclass
from functools import lru_cache

import numpy as np
import torch

RANK_SHIFT = 28
ROW_MASK = (1 << RANK_SHIFT) - 1


@dataclass(frozen=True)
class Grid:
    """Geometry shared by every layout of one model: image, window and WP grid."""
    H: int
    W: int
    ws_y: int
    ws_x: int
    wp_y: int = 1
    wp_x: int = 1
    sp: int = 1       # Ulysses sequence parallelism: every window's token sequence is cut into `sp` contiguous slices

    def __post_init__(self):
        assert self.H % self.ws_y == 0 and self.W % self.ws_x == 0, "image must be a multiple of the window"
        assert (self.H // self.ws_y) % self.wp_y == 0 and (self.W // self.ws_x) % self.wp_x == 0, \
            "window grid must divide evenly over the WP grid"
        assert (self.ws_y * self.ws_x) % self.sp == 0, "window tokens must divide evenly over the SP ranks"

    @property
    def nwy(self) -> int:
        return self.H // self.ws_y

    @property
    def nwx(self) -> int:
        return self.W // self.ws_x

    @property
    def L(self) -> int:
        return self.ws_y * self.ws_x

    @property
    def n_ranks(self) -> int:
        """Ranks that together hold one sample: WP grid x SP; rank = wp_rank * sp + sp_rank."""
        return self.wp_y * self.wp_x * self.sp

    @property
    def n_local(self) -> int:
        """Tokens of one window held by one rank."""
        return self.L // self.sp

    @property
    def nwy_loc(self) -> int:
        return self.nwy // self.wp_y

    @property
    def nwx_loc(self) -> int:
        return self.nwx // self.wp_x

    @property
    def windows_per_rank(self) -> int:
        return self.nwy_loc * self.nwx_loc

    @property
    def tokens_per_rank(self) -> int:
        """Tokens of ONE sample held by one rank."""
        return self.windows_per_rank * self.n_local

    def rank_coords(self, rank: int) -> tuple[int, int]:
        wp_rank = rank // self.sp
        return wp_rank // self.wp_x, wp_rank % self.wp_x

    def half_shift(self) -> tuple[int, int]:
        return self.ws_y // 2, self.ws_x // 2


@lru_cache(maxsize=64)
def pixel_owner(grid: Grid, shift: tuple[int, int]) -> tuple[np.ndarray, np.ndarray]:
    """For every pixel (y, x): the rank that holds it in the layout with window offset ``shift`` and its row
    index inside that rank's single-sample token block. Returns two int64 arrays of shape [H, W]."""
    sy, sx = shift
    y = (np.arange(grid.H) - sy) % grid.H
    x = (np.arange(grid.W) - sx) % grid.W
    wy, iy = y // grid.ws_y, y % grid.ws_y
    wx, ix = x // grid.ws_x, x % grid.ws_x
    ry, lwy = wy // grid.nwy_loc, wy % grid.nwy_loc
    rx, lwx = wx // grid.nwx_loc, wx % grid.nwx_loc
    seq = iy[:, None] * grid.ws_x + ix[None, :]            # position in the window's token sequence
    sp_rank, tok = seq // grid.n_local, seq % grid.n_local
    rank = (ry[:, None] * grid.wp_x + rx[None, :]) * grid.sp + sp_rank
    row = (lwy[:, None] * grid.nwx_loc + lwx[None, :]) * grid.n_local + tok
    return rank.astype(np.int64), row.astype(np.int64)


@lru_cache(maxsize=64)
def rank_pixels(grid: Grid, shift: tuple[int, int], rank: int) -> tuple[np.ndarray, np.ndarray]:
    """Pixel coordinates (y, x) of every row of ``rank``'s single-sample token block, in row order."""
    owner, row = pixel_owner(grid, shift)
    ys, xs = np.nonzero(owner == rank)
    order = np.argsort(row[ys, xs], kind="stable")
    return ys[order], xs[order]


def gather_table(grid: Grid, src_shift: tuple[int, int], dst_shift: tuple[int, int], rank: int,
                 batch: int = 1) -> torch.Tensor:
    """uint32 codes (stored as int32 bits) ``[batch * tokens_per_rank]``: where each destination row of ``rank`` in
    the ``dst_shift`` layout lives in the ``src_shift`` layout: ``(src_rank << 28) | (b * tokens_per_rank + row)``."""
    ys, xs = rank_pixels(grid, dst_shift, rank)
    owner, row = pixel_owner(grid, src_shift)
    src_rank, src_row = owner[ys, xs], row[ys, xs]
    tpr = grid.tokens_per_rank
    assert batch * tpr <= ROW_MASK, "rows per rank exceed the 28-bit row field"
    codes = []
    for b in range(batch):
        codes.append((src_rank << RANK_SHIFT) | (src_row + b * tpr))
    out = np.concatenate(codes).astype(np.uint32)
    return torch.from_numpy(out.view(np.int32).copy())


def decode_table(codes: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    u = codes.to(torch.int64) & 0xFFFFFFFF
    return u >> RANK_SHIFT, u & ROW_MASK


def apply_gather_reference(table: torch.Tensor, sources: list[torch.Tensor]) -> torch.Tensor:
    """Plain PyTorch gather through a table (CPU oracle and test reference): ``sources[r]`` is rank r's buffer."""
    rank, row = decode_table(table)
    out = torch.empty((table.numel(),) + tuple(sources[0].shape[1:]), dtype=sources[0].dtype,
                      device=sources[0].device)
    for r in range(len(sources)):
        sel = rank == r
        if sel.any():
            out[sel] = sources[r][row[sel].to(sources[r].device)]
    return out


def image_to_tokens(img: torch.Tensor, grid: Grid, shift: tuple[int, int], rank: int = 0) -> torch.Tensor:
    """``img [B, H, W, C]`` -> this rank's token rows ``[B * tokens_per_rank, C]`` in the ``shift`` layout."""
    ys, xs = rank_pixels(grid, shift, rank)
    ys_t = torch.from_numpy(ys).to(img.device)
    xs_t = torch.from_numpy(xs).to(img.device)
    B = img.shape[0]
    return img[:, ys_t, xs_t].reshape(B * ys.size, img.shape[-1])


def tokens_to_image(tok_per_rank: list[torch.Tensor], grid: Grid, shift: tuple[int, int], batch: int) -> torch.Tensor:
    """Inverse of :func:`image_to_tokens` given every rank's rows."""
    C = tok_per_rank[0].shape[-1]
    img = torch.empty((batch, grid.H, grid.W, C), dtype=tok_per_rank[0].dtype, device=tok_per_rank[0].device)
    for r, tok in enumerate(tok_per_rank):
        ys, xs = rank_pixels(grid, shift, r)
        ys_t = torch.from_numpy(ys).to(tok.device)
        xs_t = torch.from_numpy(xs).to(tok.device)
        img[:, ys_t, xs_t] = tok.reshape(batch, ys.size, C)
    return img


def halo_fraction(grid: Grid) -> float:
    """Fraction of a rank's rows that come from other ranks when moving to the shifted layout."""
    if grid.n_ranks == 1:
        return 0.0
    t = gather_table(grid, (0, 0), grid.half_shift(), 0)
    rank, _ = decode_table(t)
    return float((rank != 0).float().mean())
