"""Rank-aware logging and small output helpers.

Reference: src/aeris/utils/io.py:28-185 — ``log0`` (rank-0 logger keyed by the caller), ``print0``,
``compress_variables`` (group ``name_level`` channels into one array per variable with a level axis),
``create_empty_zarr`` / ``create_empty_numpy`` (pre-allocated rollout outputs).
"""
from __future__ import annotations

import inspect
import logging
import os
import re
import sys

import numpy as np

_LOGGERS: dict[str, logging.Logger] = {}


def get_rank() -> int:
    try:
        import torch.distributed as dist
        if dist.is_available() and dist.is_initialized():
            return dist.get_rank()
    except Exception:
        pass
    return int(os.environ.get("RANK", 0))


def _logger(name: str) -> logging.Logger:
    if name not in _LOGGERS:
        lg = logging.getLogger(f"aeris.{name}")
        if not lg.handlers:
            h = logging.StreamHandler(sys.stdout)
            h.setFormatter(logging.Formatter("[%(asctime)s][%(levelname)s][%(name)s] %(message)s", "%H:%M:%S"))
            lg.addHandler(h)
            lg.setLevel(logging.INFO)
            lg.propagate = False
        _LOGGERS[name] = lg
    return _LOGGERS[name]


def log0(msg: str, level: str = "info", rank: int = 0) -> None:
    """Log on one rank only, under a logger named after the calling module."""
    if get_rank() != rank:
        return
    frame = inspect.stack()[1]
    mod = os.path.splitext(os.path.basename(frame.filename))[0]
    getattr(_logger(mod), level)(msg)


def print0(*args, rank: int = 0, **kw) -> None:
    if get_rank() == rank:
        print(*args, flush=True, **kw)


def compress_variables(variables: list[str]) -> dict[str, tuple[list[int], list[int]]]:
    """``['2m_temperature', 'geopotential_50', 'geopotential_100', ...]`` ->
    ``{'2m_temperature': ([0], []), 'geopotential': ([4, 5, ...], [50, 100, ...]), ...}`` (channel indices, levels)."""
    out: dict[str, tuple[list[int], list[int]]] = {}
    for i, v in enumerate(variables):
        m = re.match(r"^(.*)_(\d+)$", v)
        if m and not v.startswith(("2m_", "10m_")):
            name, lvl = m.group(1), int(m.group(2))
            idx, lv = out.setdefault(name, ([], []))
            idx.append(i)
            lv.append(lvl)
        else:
            out[v] = ([i], [])
    return out


def create_empty_numpy(path: str, shape: tuple[int, ...], dtype=np.float32) -> np.memmap:
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    return np.lib.format.open_memmap(path, mode="w+", dtype=dtype, shape=shape)


def create_empty_zarr(path: str, variables: list[str], n_time: int, n_members: int, lat: int = 720, lon: int = 1440):
    """Pre-allocates a WeatherBench-style Zarr group (one array per variable, ``[member, time, (level,) lat, lon]``).
    Needs the ``zarr`` package."""
    try:
        import zarr  # type: ignore
    except Exception as e:  # pragma: no cover
        raise RuntimeError("create_empty_zarr needs the `zarr` package, which is not installed here") from e
    root = zarr.open_group(path, mode="w")
    for name, (idx, levels) in compress_variables(variables).items():
        shape = (n_members, n_time, len(levels), lat, lon) if levels else (n_members, n_time, lat, lon)
        chunks = (1, 1, len(levels), lat, lon) if levels else (1, 1, lat, lon)
        root.zeros(name, shape=shape, chunks=chunks, dtype="f4")
    return root
