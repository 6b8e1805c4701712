"""Render rollout fields to an animated GIF on the CPU (matplotlib Agg backend; no GL, no display).

Reference: scripts/animate.py:74-137, 189-232 (matplotlib + cartopy FuncAnimation from HDF5 rollouts). matplotlib and
cartopy are optional dependencies: the script imports them lazily and says so when one is missing. Without cartopy the fields
are drawn on a plain equirectangular axis.

    python -m aeris_gb_b200.cli.animate --input rollout.npy --variable 2m_temperature --out t2m.gif
"""
from __future__ import annotations

import argparse

import numpy as np

from ..data.era5 import variable_names
from ..data.store import open_array


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--input", required=True, help="[time, C, H, W] array file")
    ap.add_argument("--variable", default="2m_temperature")
    ap.add_argument("--channels", type=int, default=69)
    ap.add_argument("--out", default="rollout.gif")
    ap.add_argument("--fps", type=int, default=4)
    a = ap.parse_args(argv)
    try:
        import matplotlib
        matplotlib.use("Agg")
        import matplotlib.pyplot as plt
        from matplotlib.animation import FuncAnimation, PillowWriter
    except Exception as e:
        raise SystemExit(f"animate needs matplotlib, which is not installed here ({e})")
    arr = open_array(a.input)
    ch = variable_names(a.channels).index(a.variable)
    frames = [np.asarray(arr[t, ch]) for t in range(arr.shape[0])]
    vmin, vmax = min(f.min() for f in frames), max(f.max() for f in frames)
    fig, ax = plt.subplots(figsize=(10, 5))
    im = ax.imshow(frames[0], origin="lower", extent=(0, 360, -90, 90), vmin=vmin, vmax=vmax, cmap="RdBu_r")
    fig.colorbar(im, ax=ax, shrink=0.7)

    def update(i):
        im.set_data(frames[i])
        ax.set_title(f"{a.variable}  step {i}")
        return (im,)
    FuncAnimation(fig, update, frames=len(frames), blit=False).save(a.out, writer=PillowWriter(fps=a.fps))
    print(a.out)


if __name__ == "__main__":
    main()
