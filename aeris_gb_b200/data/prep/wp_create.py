"""Create one data file per window-parallel rank from a merged ``[samples, C, 721, 1440]`` array.

Reference: scripts/data_processing/wp_create.py:14-99 — the first latitude row is dropped (720 rows remain), windows
are dealt round-robin to the WP grid (``window (wy, wx) -> rank (wy mod WP_Y, wx mod WP_X)``) and each rank's windows
are packed into ``y_{y}_x_{x}`` of shape ``[samples, C, 720/WP_Y, 1440/WP_X]``; a sample that reads back as all zeros
aborts the job (:81-84). ``--layout block`` writes contiguous blocks instead (the layout of this framework's
single-node engine and of the reference's WP-only inference).

    python -m aeris_gb_b200.data.prep.wp_create --src merged.npy --dst DIR --wp-y 4 --wp-x 4 --window 60 60
"""
from __future__ import annotations

import argparse
import os

import numpy as np

from ..store import open_array, save_array


def tile_for_rank(sample: np.ndarray, wy: int, wx: int, WP_Y: int, WP_X: int, ws_y: int, ws_x: int,
                  layout: str = "strided") -> np.ndarray:
    """sample [C, 721 or 720, 1440] -> [C, 720/WP_Y, 1440/WP_X] for rank (wy, wx)."""
    if sample.shape[1] == 721:
        sample = sample[:, 1:]
    C, H, W = sample.shape
    if layout == "block":
        hb, wb = H // WP_Y, W // WP_X
        return sample[:, wy * hb:(wy + 1) * hb, wx * wb:(wx + 1) * wb]
    win = sample.reshape(C, H // ws_y, ws_y, W // ws_x, ws_x)
    mine = win[:, wy::WP_Y, :, wx::WP_X, :]
    return mine.reshape(C, mine.shape[1] * ws_y, mine.shape[3] * ws_x)


def create(src: str, dst: str, WP_Y: int, WP_X: int, window=(60, 60), layout="strided", rank=0, world=1,
           max_samples: int | None = None) -> list[str]:
    ds = open_array(src)
    n = ds.shape[0] if max_samples is None else min(ds.shape[0], max_samples)
    coords = [(y, x) for y in range(WP_Y) for x in range(WP_X)]
    written = []
    for (y, x) in coords[rank::world]:
        out = None
        for i in range(n):
            s = np.asarray(ds[i], dtype=np.float32)
            t = tile_for_rank(s, y, x, WP_Y, WP_X, window[0], window[1], layout)
            if not np.isnan(t).all() and np.nanvar(t) == 0:
                raise RuntimeError(f"sample {i} read back with zero variance for rank ({y},{x}): bad read")
            if out is None:
                out = np.empty((n,) + t.shape, dtype=np.float32)
            out[i] = t
        written.append(save_array(os.path.join(dst, f"y_{y}_x_{x}"), out))
    return written


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--src", required=True)
    ap.add_argument("--dst", required=True)
    ap.add_argument("--wp-y", type=int, required=True)
    ap.add_argument("--wp-x", type=int, required=True)
    ap.add_argument("--window", type=int, nargs=2, default=(60, 60))
    ap.add_argument("--layout", choices=["strided", "block"], default="strided")
    ap.add_argument("--rank", type=int, default=int(os.environ.get("RANK", 0)))
    ap.add_argument("--world", type=int, default=int(os.environ.get("WORLD_SIZE", 1)))
    a = ap.parse_args()
    for p in create(a.src, a.dst, a.wp_y, a.wp_x, tuple(a.window), a.layout, a.rank, a.world):
        print(p)


if __name__ == "__main__":
    main()
