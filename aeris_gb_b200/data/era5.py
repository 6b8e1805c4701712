"""ERA5 datasets (0.25 degree, 721 x 1440, 6-hourly).

Channel sets (reference src/aeris/data/era5.py:269-275, :293): 69 = 4 surface fields + 5 variables x 13 pressure
levels; 72 adds top-of-atmosphere radiation, surface geopotential and land-sea mask; 73 additionally has sea-surface
temperature (before the radiation channel). Standardisation statistics are read from ``normalize_{mean,std}.npz`` and
``normalize_diff_{mean,std}_{interval}.npz`` in the dataset root (:310-318).

A training item is ``(standardised state [+ standardised radiation at t + dt], standardised residual X(t+dt) - X(t))``
(:373-393); SST NaNs over land are filled with the field minimum (:376-379); an inference item is ``(x, raw label
stack)`` (:396-407). Window-parallel training reads one file per WP rank, ``y_{wp_y}_x_{wp_x}`` (:346-358).
"""
from __future__ import annotations

import os

import numpy as np
import torch
from torch.utils.data import Dataset

from .store import open_array

LEVELS = [50, 100, 150, 200, 250, 300, 400, 500, 600, 700, 850, 925, 1000]
SURFACE = ["2m_temperature", "10m_u_component_of_wind", "10m_v_component_of_wind", "mean_sea_level_pressure"]
UPPER = ["geopotential", "u_component_of_wind", "v_component_of_wind", "temperature", "specific_humidity"]
STATIC = ["toa_incident_solar_radiation", "geopotential_at_surface", "land_sea_mask"]


def variable_names(n_channels: int) -> list[str]:
    names = SURFACE + [f"{v}_{l}" for v in UPPER for l in LEVELS]
    if n_channels == 69:
        return names
    if n_channels == 72:
        return names + STATIC
    if n_channels == 73:
        return names + ["sea_surface_temperature"] + STATIC
    raise ValueError(f"no channel set with {n_channels} channels")


class Standardizer:
    """Per-channel (mean, std) of the state and of the ``interval``-hour residual."""

    def __init__(self, root: str | None, variables: list[str], interval: int):
        C = len(variables)
        if root is None:
            self.x_means, self.x_stds = np.zeros((C, 1, 1), np.float32), np.ones((C, 1, 1), np.float32)
            self.t_means, self.t_stds = np.zeros((C, 1, 1), np.float32), np.ones((C, 1, 1), np.float32)
            return

        def stack(fname):
            with np.load(os.path.join(root, fname)) as d:
                return np.stack([d[v] for v in variables], axis=0).reshape(-1, 1, 1).astype(np.float32)
        self.x_means, self.x_stds = stack("normalize_mean.npz"), stack("normalize_std.npz")
        self.t_means = stack(f"normalize_diff_mean_{interval}.npz")
        self.t_stds = stack(f"normalize_diff_std_{interval}.npz")

    def standardize_x(self, x, a=0, b=None):
        return (x - self.x_means[a:b]) / self.x_stds[a:b]

    def unstandardize_x(self, x, a=0, b=None):
        return x * self.x_stds[a:b] + self.x_means[a:b]

    def standardize_t(self, t, a=0, b=None):
        return (t - self.t_means[a:b]) / self.t_stds[a:b]

    def unstandardize_t(self, t, a=0, b=None):
        return t * self.t_stds[a:b] + self.t_means[a:b]

    def tensors(self, device, a=0, b=None) -> dict[str, torch.Tensor]:
        """Channel-last [C] tensors for the on-device sampler kernels."""
        f = lambda v: torch.from_numpy(v[a:b].reshape(-1)).to(device)
        return dict(x_mean=f(self.x_means), x_std=f(self.x_stds), t_mean=f(self.t_means), t_std=f(self.t_stds))


def _fill_nan_min(a: np.ndarray, ch: int):
    sl = a[..., ch, :, :]
    if np.isnan(sl).any():
        np.copyto(sl, np.nanmin(sl), where=np.isnan(sl))


class ERA5NRMDataset(Dataset):
    """Monolithic pre-processed dataset ``[samples, C, H, W]``, optionally one file per WP rank."""

    def __init__(self, root: str | None, path: str, interval: int = 6, channels: int = 69, test: bool = False,
                 samples: int | None = None, inference: bool = False):
        self.root, self.path, self.interval, self.channels, self.inference = root, path, interval, channels, inference
        self.dt = interval // 6
        self.variables = variable_names(channels)
        self.stats = Standardizer(root, self.variables, interval)
        self._samples = samples
        self._default_samples = (1464 if test else 58440) - self.dt
        self.ds = None
        self.benchmark = False
        self.load_t, self.load_inf_labels = True, 0
        self.n_state = 69 if channels == 69 else self.variables.index("toa_incident_solar_radiation")

    n_channels = property(lambda self: self.channels)
    img_resolution = property(lambda self: (721, 1440))

    def get_lat_lon(self) -> tuple[np.ndarray, np.ndarray]:
        """``lat.npy`` / ``lon.npy`` of the statistics folder (src/aeris/data/era5.py:300-303)."""
        return (np.load(os.path.join(self.root, "lat.npy")).astype(np.float32),
                np.load(os.path.join(self.root, "lon.npy")).astype(np.float32))

    def get_time(self, idx: int, start: str = "1979-01-01T00", step_hours: int = 6) -> np.datetime64:
        """Valid time of sample ``idx``. The monolithic array carries no time stamps (the reference reads them from its
        per-step files, :338-341), so the time follows from the index on the 6-hourly axis that starts at ``start``."""
        return np.datetime64(start) + np.timedelta64(int(idx) * step_hours, "h")

    def __len__(self):
        if self._samples is not None:
            return self._samples
        return (self.ds.shape[0] - self.dt) if self.ds is not None else self._default_samples

    def open_file(self, wp_y_rank: int | None = None, wp_x_rank: int | None = None, load_x=True, load_t=True,
                  load_inf_labels: int = 0, benchmark: bool = False):
        p = self.path if wp_y_rank is None else os.path.join(self.path, f"y_{wp_y_rank}_x_{wp_x_rank}")
        self.ds = open_array(p)
        self.load_t, self.load_inf_labels, self.benchmark = load_t, load_inf_labels, benchmark
        if benchmark:
            self.ds = np.asarray(self.ds[:104])       # preload, then cycle over the first 100 samples (:357-358,:364)

    def __getitem__(self, idx: int):
        if self.benchmark:
            idx = idx % 100
        s = self.stats
        x = np.array(self.ds[idx], dtype=np.float32)
        if self.channels == 73:
            _fill_nan_min(x, self.variables.index("sea_surface_temperature"))
        if self.load_inf_labels > 0:
            labels = np.array(self.ds[idx: idx + (self.load_inf_labels + 1) * self.dt: self.dt], dtype=np.float32)
            if self.channels == 73:
                _fill_nan_min(labels, self.variables.index("sea_surface_temperature"))
            xs = s.standardize_x(x)
            if self.channels > 69:
                rad = self.variables.index("toa_incident_solar_radiation")
                nxt = np.array(self.ds[idx + self.dt, rad:rad + 1], dtype=np.float32)
                xs = np.concatenate([xs, s.standardize_x(nxt, rad, rad + 1)], axis=0)
            return torch.from_numpy(xs).float(), torch.from_numpy(labels)
        if not self.load_t:
            return torch.from_numpy(s.standardize_x(x)).float()
        t = np.array(self.ds[idx + self.dt], dtype=np.float32)
        if self.channels > 69:
            rad = self.variables.index("toa_incident_solar_radiation")
            if self.channels == 73:
                _fill_nan_min(t, self.variables.index("sea_surface_temperature"))
            extra = s.standardize_x(t[rad:rad + 1], rad, rad + 1)
            xs = np.concatenate([s.standardize_x(x), extra], axis=0)       # state + radiation at t + dt
            res = s.standardize_t(t[:rad] - x[:rad], 0, rad)
            return torch.from_numpy(xs).float(), torch.from_numpy(res).float()
        return torch.from_numpy(s.standardize_x(x)).float(), torch.from_numpy(s.standardize_t(t - x)).float()


class ERA5NRMRTIDataset(ERA5NRMDataset):
    """Random-time-interval variant: each item draws an interval from ``intervals`` hours and returns it with the
    pair; in benchmark mode the data are synthetic N(0,1) of ``data_shape`` (reference :125-245, :201-205)."""

    def __init__(self, *a, intervals=(6, 12, 24), seed: int = 0, **kw):
        super().__init__(*a, **kw)
        self.intervals = tuple(intervals)
        self.dt = max(self.intervals) // 6
        self._rng = np.random.default_rng(seed)
        self._synthetic = None

    def open_file(self, wp_y_rank=None, wp_x_rank=None, load_x=True, load_t=True, load_inf_labels=0,
                  benchmark=False, data_shape=None):
        if benchmark:
            shape = tuple(data_shape or (30, 69, 720, 1440))
            g = torch.Generator().manual_seed(1234)
            self._synthetic = torch.randn(shape, generator=g)
            self.benchmark, self.load_t = True, load_t
            self._samples = shape[0] - self.dt
            return
        super().open_file(wp_y_rank, wp_x_rank, load_x, load_t, load_inf_labels, False)

    def __getitem__(self, idx: int):
        hours = int(self._rng.choice(self.intervals))
        k = hours // 6
        interval = torch.tensor([float(hours)])
        if self._synthetic is not None:
            i = idx % (self._synthetic.shape[0] - self.dt)
            return self._synthetic[i], self._synthetic[i + k], interval
        x = np.array(self.ds[idx], dtype=np.float32)
        t = np.array(self.ds[idx + k], dtype=np.float32)
        s = self.stats
        return (torch.from_numpy(s.standardize_x(x)).float(), torch.from_numpy(s.standardize_x(t)).float(), interval)


class ERA5Dataset(Dataset):
    """Legacy layout: one array file per time step in ``root/<split>/`` (reference :18-123)."""

    def __init__(self, root: str, split: str = "train", interval: int = 6, channels: int = 69):
        self.dir = os.path.join(root, split)
        self.files = sorted(f for f in os.listdir(self.dir) if f.endswith((".npy", ".h5", ".hdf5")))
        self.dt = interval // 6
        self.variables = variable_names(channels)
        self.stats = Standardizer(root, self.variables, interval)

    def __len__(self):
        return len(self.files) - self.dt

    def _read(self, i):
        return np.asarray(open_array(os.path.join(self.dir, self.files[i]))[...], dtype=np.float32)

    def __getitem__(self, idx):
        x, t = self._read(idx), self._read(idx + self.dt)
        return (torch.from_numpy(self.stats.standardize_x(x)).float(),
                torch.from_numpy(self.stats.standardize_t(t - x)).float())


class ERA5InferenceDataset(Dataset):
    """Monolithic test-year file ``[1464, 73, 721, 1440]``: item = (state at idx, states at idx + k*dt for the
    rollout); SST NaNs are filled per 4x4 tile with the tile minimum where a tile has any sea, else with the global
    minimum (reference src/aeris_wp_inference/era5.py:31-156, :136-146)."""

    def __init__(self, root: str | None, path: str, interval: int = 6, channels: int = 73, rollout_steps: int = 0):
        self.variables = variable_names(channels)
        self.stats = Standardizer(root, self.variables, interval)
        self.ds = open_array(path)
        self.dt, self.steps, self.channels = interval // 6, rollout_steps, channels

    def __len__(self):
        return self.ds.shape[0] - self.dt * max(self.steps, 1)

    def fill_sst(self, a: np.ndarray) -> np.ndarray:
        if self.channels != 73:
            return a
        ch = self.variables.index("sea_surface_temperature")
        sst = a[..., ch, :, :]
        if not np.isnan(sst).any():
            return a
        H, W = sst.shape[-2:]
        h4, w4 = H - H % 4, W - W % 4
        tiles = sst[..., :h4, :w4].reshape(*sst.shape[:-2], h4 // 4, 4, w4 // 4, 4)
        with np.errstate(all="ignore"):
            tmin = np.nanmin(tiles, axis=(-3, -1), keepdims=True)
        gmin = np.nanmin(sst)
        fill = np.where(np.isnan(tmin), gmin, tmin)
        filled = np.where(np.isnan(tiles), fill, tiles).reshape(*sst.shape[:-2], h4, w4)
        sst[..., :h4, :w4] = filled
        np.copyto(sst, gmin, where=np.isnan(sst))
        return a

    def __getitem__(self, idx):
        x = self.fill_sst(np.array(self.ds[idx], dtype=np.float32))
        labels = self.fill_sst(np.array(self.ds[idx: idx + (self.steps + 1) * self.dt: self.dt], dtype=np.float32))
        return torch.from_numpy(self.stats.standardize_x(x)).float(), torch.from_numpy(labels)
