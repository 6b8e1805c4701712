"""Array storage behind the datasets: HDF5 through ``h5py`` when it is installed, ``.npy`` memory maps otherwise.

The reference reads HDF5 only (src/aeris/data/era5.py:346-358). h5py is an optional dependency, so every dataset goes
through :func:`open_array`, which accepts ``file.hdf5`` (dataset name ``input``) or ``file.npy`` and returns an object
with ``shape`` and numpy-style indexing. :func:`save_array` writes the format the current environment can read back.
"""
from __future__ import annotations

import os

import numpy as np

try:  # optional
    import h5py  # type: ignore
    HAVE_H5 = True
except Exception:  # pragma: no cover - depends on the image
    h5py = None
    HAVE_H5 = False


class H5Array:
    def __init__(self, path: str, name: str = "input"):
        self.file = h5py.File(path, "r")
        self.ds = self.file[name]
        self.shape = self.ds.shape

    def __getitem__(self, idx):
        return np.asarray(self.ds[idx])

    def close(self):
        self.file.close()


def resolve(path: str) -> str:
    """Picks the existing variant of ``path`` among .hdf5 / .h5 / .npy (given with or without extension)."""
    stem = path
    for ext in (".hdf5", ".h5", ".npy"):
        if path.endswith(ext):
            stem = path[:-len(ext)]
    cands = ([stem + ".hdf5", stem + ".h5"] if HAVE_H5 else []) + [stem + ".npy"]
    for c in cands:
        if os.path.exists(c):
            return c
    raise FileNotFoundError(f"none of {cands} exists" + ("" if HAVE_H5 else " (h5py is not installed: HDF5 files cannot be read)"))


def open_array(path: str, name: str = "input"):
    p = resolve(path)
    if p.endswith(".npy"):
        return np.load(p, mmap_mode="r")
    return H5Array(p, name)


def save_array(path_stem: str, arr: np.ndarray, name: str = "input", prefer_h5: bool = True) -> str:
    os.makedirs(os.path.dirname(os.path.abspath(path_stem)), exist_ok=True)
    if HAVE_H5 and prefer_h5:
        p = path_stem + ".hdf5"
        with h5py.File(p, "w") as f:
            f.create_dataset(name, data=arr)
        return p
    p = path_stem + ".npy"
    np.save(p, arr)
    return p
