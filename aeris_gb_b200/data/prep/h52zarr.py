"""Convert rollout output files to a WeatherBench-style Zarr store.

Reference: scripts/data_processing/bh52zarr_dist.py:126-262 with a dask-distributed cluster started by
``dask-launch.sh`` and a 10x retry loop around each write. The conversion needs ``zarr`` (and optionally ``dask``);
both are optional dependencies: the module imports them lazily and the CLI reports what is missing. The
chunked copy itself is a plain loop over (member, time) slabs that worker processes split by ``--rank/--world``.

    python -m aeris_gb_b200.data.prep.h52zarr --src rollout_dir --dst out.zarr --variables-from 73
"""
from __future__ import annotations

import argparse
import os
import time

import numpy as np

from ...utils.io import compress_variables
from ..era5 import variable_names
from ..store import open_array


def convert(src_files: list[str], dst: str, variables: list[str], rank: int = 0, world: int = 1, retries: int = 10):
    try:
        import zarr  # type: ignore
    except Exception as e:  # pragma: no cover - depends on the image
        raise RuntimeError("h52zarr needs the `zarr` package, which is not installed here") from e
    groups = compress_variables(variables)
    root = zarr.open_group(dst, mode="a")
    for fi, f in enumerate(src_files):
        if fi % world != rank:
            continue
        arr = open_array(f)                     # [time, C, H, W]
        for name, (idx, levels) in groups.items():
            data = np.asarray(arr[:, idx]) if levels else np.asarray(arr[:, idx[0]])
            for attempt in range(retries):      # shared file systems fail transiently; the reference retries 10x
                try:
                    root.require_group(f"member_{fi}").array(name, data, overwrite=True)
                    break
                except Exception:
                    if attempt == retries - 1:
                        raise
                    time.sleep(1.0 + attempt)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--src", required=True)
    ap.add_argument("--dst", required=True)
    ap.add_argument("--variables-from", type=int, default=70, help="channel-set size (69, 70, 72 or 73)")
    ap.add_argument("--rank", type=int, default=int(os.environ.get("RANK", 0)))
    ap.add_argument("--world", type=int, default=int(os.environ.get("WORLD_SIZE", 1)))
    a = ap.parse_args()
    n = a.variables_from
    variables = variable_names(73)[:70] if n == 70 else variable_names(n)
    files = sorted(os.path.join(a.src, f) for f in os.listdir(a.src) if f.endswith((".npy", ".h5", ".hdf5")))
    convert(files, a.dst, variables, a.rank, a.world)


if __name__ == "__main__":
    main()
