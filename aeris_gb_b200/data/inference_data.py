"""Initial conditions, forcings and verification fields of the inference entry points, read from a test file.

Reference: the strided initial conditions split over the data-parallel ranks (src/aeris/pp_generate.py:611-637,
src/aeris_wp_inference/inference.py:302-314), the per-step forcings ``radiation(T + k), surface geopotential,
land-sea mask, radiation(T + k + 1)`` appended to the condition (pp_generate.py:291-297, inference.py:130), the
north-pole row dropped (src/aeris_wp_inference/era5.py:281-283), the state advanced in physical units and
re-standardised with the dataset statistics (pp_generate.py:325-333), and the rollout written per window-parallel tile
(pp_generate.py:93-99, 474-479). The reference loads every sample on one rank and scatters it over a gloo side group
(era5.py:249-277); here every rank memory-maps the file and cuts its own block.

File layout: ``[T, 73, H + 1, W]`` (69 atmospheric channels, sea-surface temperature, radiation, surface geopotential,
land-sea mask; first latitude row = north pole), or ``[T, 73, H, W]`` when the pole row is already gone.
"""
from __future__ import annotations

import os

import numpy as np
import torch

from .era5 import ERA5InferenceDataset
from .store import save_array


def strided_indices(n_times: int, steps: int, dt: int, stride: int, dp_rank: int, dp: int, start: int = 0,
                    end: int | None = None) -> tuple[list[int], list[int]]:
    """(all strided initial-condition indices, this data-parallel rank's share). Every initial condition leaves room
    for ``steps`` forecast steps of ``dt`` samples; the share is every ``dp``-th index starting at ``dp_rank``."""
    last = n_times - steps * dt if end is None else min(end + 1, n_times - steps * dt)
    all_ic = list(range(start, max(last, start), stride))
    return all_ic, all_ic[dp_rank::dp]


class InferenceData:
    """One rank's view of the test file: block ``wp_rank`` of a ``wp`` grid of the ``img`` = (H, W) model grid."""

    def __init__(self, path: str, root: str | None, img: tuple[int, int], wp: tuple[int, int] = (1, 1),
                 wp_rank: tuple[int, int] = (0, 0), interval: int = 6, rollout_steps: int = 1,
                 out_channels: int = 70, channels: int = 73):
        self.ds = ERA5InferenceDataset(root, path, interval, channels, rollout_steps)
        self.img, self.wp, self.wp_rank, self.steps, self.C = img, wp, wp_rank, rollout_steps, out_channels
        rows = self.ds.ds.shape[-2]
        assert rows in (img[0], img[0] + 1) and self.ds.ds.shape[-1] == img[1], \
            f"file grid {self.ds.ds.shape[-2:]} does not fit the model grid {img}"
        self.row0 = rows - img[0]                       # 1: drop the north-pole row
        v = self.ds.variables
        self.i_rad = v.index("toa_incident_solar_radiation") if channels > 69 else None
        self.i_gp = v.index("geopotential_at_surface") if channels > 69 else None
        self.i_lsm = v.index("land_sea_mask") if channels > 69 else None
        self.n_forcing = 4 if channels > 69 else 0
        self.dt = self.ds.dt

    def __len__(self) -> int:
        return len(self.ds)

    def _block(self, a: np.ndarray) -> torch.Tensor:
        """[..., C, rows, W] array -> this rank's [..., hb, wb, C] block as a tensor."""
        hb, wb = self.img[0] // self.wp[0], self.img[1] // self.wp[1]
        y, x = self.wp_rank
        blk = a[..., self.row0 + y * hb:self.row0 + (y + 1) * hb, x * wb:(x + 1) * wb]
        return torch.from_numpy(np.ascontiguousarray(np.moveaxis(blk, -3, -1))).float()

    def stats(self, device) -> dict[str, torch.Tensor]:
        return self.ds.stats.tensors(device, 0, self.C)

    def sample(self, idx: int) -> dict:
        """Initial condition ``idx``: ``state`` [hb, wb, C] in physical units, ``forcing`` [steps, hb, wb, 4]
        standardised (radiation at step k, surface geopotential, land-sea mask, radiation at step k + 1),
        ``truth`` [steps, hb, wb, C] physical states at the verification times."""
        x_std, labels = self.ds[idx]                                  # [73, rows, W] standardised, [steps+1, 73, ...] raw
        labels = labels.numpy()
        s = self.ds.stats
        out = {"state": self._block(labels[0, :self.C]), "truth": self._block(labels[1:, :self.C])}
        if self.n_forcing:
            r = self.i_rad
            rad = s.standardize_x(labels[:, r:r + 1], r, r + 1)         # [steps+1, 1, rows, W]
            xs = x_std.numpy()
            static = np.concatenate([xs[self.i_gp:self.i_gp + 1], xs[self.i_lsm:self.i_lsm + 1]], axis=0)
            static = np.broadcast_to(static, (self.steps, *static.shape))
            forcing = np.concatenate([rad[:-1], static, rad[1:]], axis=1)   # [steps, 4, rows, W]
            out["forcing"] = self._block(forcing)
        else:
            out["forcing"] = None
        return out


class RolloutWriter:
    """Per-rank rollout file ``<stem>_y{wp_y}_x{wp_x}``: ``[initial conditions, steps + 1, members, C, hb, wb]`` in
    physical units, index 0 = the initial state (the reference's per-tile slab of pp_generate.py:93-99)."""

    def __init__(self, out_dir: str, stem: str, wp_rank: tuple[int, int], n_ic: int, steps: int, members: int, C: int,
                 hb: int, wb: int):
        os.makedirs(out_dir, exist_ok=True)
        self.path_stem = os.path.join(out_dir, f"{stem}_y{wp_rank[0]}_x{wp_rank[1]}")
        self.buf = np.zeros((n_ic, steps + 1, members, C, hb, wb), dtype=np.float32)

    def put(self, ic: int, step: int, members_state: torch.Tensor) -> None:
        """members_state [M, hb, wb, C] (physical units) for forecast step ``step`` (0 = initial state)."""
        self.buf[ic, step] = members_state.detach().float().cpu().permute(0, 3, 1, 2).numpy()

    def close(self) -> str:
        return save_array(self.path_stem, self.buf)
