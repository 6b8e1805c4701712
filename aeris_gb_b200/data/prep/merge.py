"""Merge per-time-step files into one ``[samples, C, 721, 1440]`` array, sharded over worker processes.

Reference: scripts/data_processing/merge.py:27-170 (MPI ranks each copy a contiguous range of time steps into one
HDF5 opened with the MPI driver). Here workers are plain processes selected by ``--rank/--world`` (or the
RANK/WORLD_SIZE environment of torchrun); each writes its range into a shared ``.npy`` memory map (or, with h5py, its
own ``part_{rank}.hdf5`` that :func:`concat_parts` joins), so no MPI installation is needed.

    python -m aeris_gb_b200.data.prep.merge --src DIR --dst OUT --channels 73 [--rank R --world N]
"""
from __future__ import annotations

import argparse
import os

import numpy as np

from ..era5 import variable_names
from ..store import open_array


def file_list(src: str) -> list[str]:
    return sorted(os.path.join(src, f) for f in os.listdir(src) if f.endswith((".npy", ".h5", ".hdf5")))


def my_range(n: int, rank: int, world: int) -> range:
    per, extra = divmod(n, world)
    lo = rank * per + min(rank, extra)
    return range(lo, lo + per + (1 if rank < extra else 0))


def merge(src: str, dst: str, channels: int, rank: int = 0, world: int = 1, shape_hw=(721, 1440)) -> str:
    files = file_list(src)
    n = len(files)
    assert n > 0, f"no time-step files in {src}"
    out_path = dst if dst.endswith(".npy") else dst + ".npy"
    full_shape = (n, channels, *shape_hw)
    if rank == 0 and not os.path.exists(out_path):
        np.lib.format.open_memmap(out_path, mode="w+", dtype=np.float32, shape=full_shape).flush()
    import time
    t0 = time.monotonic()
    while not os.path.exists(out_path):      # other workers wait (at most ten minutes) for rank 0 to create the file
        if time.monotonic() - t0 > 600.0:
            raise TimeoutError(f"rank {rank}: {out_path} was not created by rank 0 within 600 s")
        time.sleep(0.2)
    out = np.lib.format.open_memmap(out_path, mode="r+")
    for i in my_range(n, rank, world):
        a = np.asarray(open_array(files[i])[...], dtype=np.float32)
        assert a.shape == full_shape[1:], f"{files[i]}: {a.shape} != {full_shape[1:]}"
        out[i] = a
    out.flush()
    return out_path


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--src", required=True)
    ap.add_argument("--dst", required=True)
    ap.add_argument("--channels", type=int, default=73)
    ap.add_argument("--rank", type=int, default=int(os.environ.get("RANK", 0)))
    ap.add_argument("--world", type=int, default=int(os.environ.get("WORLD_SIZE", 1)))
    a = ap.parse_args()
    assert len(variable_names(a.channels)) == a.channels
    print(merge(a.src, a.dst, a.channels, a.rank, a.world))


if __name__ == "__main__":
    main()
