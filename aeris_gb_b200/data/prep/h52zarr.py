"""Convert rollout output files to a WeatherBench-style Zarr store.

Reference: scripts/data_processing/bh52zarr_dist.py:126-262 with a dask-distributed cluster started by
``dask-launch.sh`` and a 10x retry loop around each write. Here worker processes split the files by
``--rank/--world`` (no dask), every write is retried, and the store is written by the ``zarr`` package when it is
installed, otherwise by a built-in writer of the Zarr v2 directory format (uncompressed chunks).

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


class ZarrV2Writer:
    """Minimal writer of the Zarr v2 directory format (uncompressed little-endian chunks, C order): a ``.zgroup`` per
    group, and per array a ``.zarray`` with shape / chunks / dtype, a ``.zattrs`` with xarray's ``_ARRAY_DIMENSIONS``,
    and one file per chunk named by its dot-separated chunk index. Stores written this way open with ``zarr`` and
    ``xarray.open_zarr``; it is used when the ``zarr`` package is absent."""

    def __init__(self, root: str):
        self.root = root
        self._group(root)

    @staticmethod
    def _group(path: str):
        import json
        os.makedirs(path, exist_ok=True)
        with open(os.path.join(path, ".zgroup"), "w") as f:
            json.dump({"zarr_format": 2}, f)

    def write(self, group: str, name: str, data: np.ndarray, dims: list[str], time_chunk: int = 1):
        import json
        gpath = os.path.join(self.root, group)
        self._group(gpath)
        apath = os.path.join(gpath, name)
        os.makedirs(apath, exist_ok=True)
        data = np.ascontiguousarray(data, dtype="<f4")
        chunks = [min(time_chunk, data.shape[0])] + list(data.shape[1:])
        with open(os.path.join(apath, ".zarray"), "w") as f:
            json.dump({"zarr_format": 2, "shape": list(data.shape), "chunks": chunks, "dtype": "<f4", "compressor": None,
                       "fill_value": 0.0, "order": "C", "filters": None}, f)
        with open(os.path.join(apath, ".zattrs"), "w") as f:
            json.dump({"_ARRAY_DIMENSIONS": dims}, f)
        tail = ".".join(["0"] * (data.ndim - 1))
        for ci, t0 in enumerate(range(0, data.shape[0], chunks[0])):
            block = data[t0:t0 + chunks[0]]
            if block.shape[0] < chunks[0]:                       # edge chunks are stored full size
                pad = np.zeros((chunks[0] - block.shape[0], *block.shape[1:]), dtype="<f4")
                block = np.concatenate([block, pad])
            fname = f"{ci}.{tail}" if tail else f"{ci}"
            tmp = os.path.join(apath, fname + ".tmp")
            with open(tmp, "wb") as f:
                f.write(block.tobytes())
            os.replace(tmp, os.path.join(apath, fname))


def read_zarr_v2_array(path: str) -> np.ndarray:
    """Reads back an uncompressed Zarr v2 array directory (what :class:`ZarrV2Writer` writes)."""
    import json
    meta = json.load(open(os.path.join(path, ".zarray")))
    shape, chunks = meta["shape"], meta["chunks"]
    out = np.zeros(shape, dtype=meta["dtype"])
    tail = ".".join(["0"] * (len(shape) - 1))
    for ci, t0 in enumerate(range(0, shape[0], chunks[0])):
        fname = f"{ci}.{tail}" if tail else f"{ci}"
        block = np.frombuffer(open(os.path.join(path, fname), "rb").read(), dtype=meta["dtype"]).reshape(chunks)
        out[t0:t0 + chunks[0]] = block[:shape[0] - t0]
    return out


def _write_with_retries(write, retries: int, sleep=time.sleep):
    """Shared file systems fail transiently; the reference retries every write ten times."""
    for attempt in range(retries):
        try:
            return write()
        except Exception:
            if attempt == retries - 1:
                raise
            sleep(1.0 + attempt)


def convert(src_files: list[str], dst: str, variables: list[str], rank: int = 0, world: int = 1, retries: int = 10,
            use_zarr_package: bool | None = None, sleep=time.sleep):
    """One group ``member_{i}`` per rollout file ``[time, C, H, W]``; multi-level variables become
    ``[time, level, latitude, longitude]`` arrays, surface variables ``[time, latitude, longitude]``. Worker
    ``rank`` of ``world`` converts every ``world``-th file. With the ``zarr`` package installed (and
    ``use_zarr_package`` not False) it does the writing; otherwise the built-in Zarr v2 writer."""
    zarr = None
    if use_zarr_package is not False:
        try:
            import zarr  # type: ignore
        except Exception:
            if use_zarr_package:
                raise RuntimeError("h52zarr was asked to use the `zarr` package, which is not installed")
    groups = compress_variables(variables)
    root = zarr.open_group(dst, mode="a") if zarr is not None else None
    writer = ZarrV2Writer(dst) if zarr is None else None
    for fi, f in enumerate(src_files):
        if fi % world != rank:
            continue
        arr = open_array(f)                     # [time, C, H, W]
        for name, (idx, levels) in groups.items():
            data = np.asarray(arr[:, idx]) if levels else np.asarray(arr[:, idx[0]])
            dims = ["time", "level", "latitude", "longitude"] if levels else ["time", "latitude", "longitude"]
            if zarr is not None:
                _write_with_retries(lambda: root.require_group(f"member_{fi}").array(name, data, overwrite=True),
                                    retries, sleep)
            else:
                _write_with_retries(lambda: writer.write(f"member_{fi}", name, data, dims), retries, sleep)


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
