"""Synthetic standardised fields: i.i.d. N(0,1) per channel, deterministic in (seed, index), generated for one WP
rank's block only. Used by the benchmarks (no dataset can be downloaded) and by the reference's own benchmark mode
(src/aeris/data/era5.py:201-205 uses ``torch.randn(data_shape)``)."""
from __future__ import annotations

import torch
from torch.utils.data import Dataset


class SyntheticERA5(Dataset):
    def __init__(self, img=(720, 1440), cond_channels=74, target_channels=70, wp=(1, 1), wp_rank=(0, 0),
                 length: int = 4096, seed: int = 0, pool: int = 4, channels_last: bool = True,
                 intervals: tuple | None = None):
        self.hb, self.wb = img[0] // wp[0], img[1] // wp[1]
        self.cc, self.ct, self.length, self.seed, self.pool = cond_channels, target_channels, length, seed, pool
        self.rank_id = wp_rank[0] * wp[1] + wp_rank[1]
        self.channels_last = channels_last
        # random-time-interval training (reference ERA5NRMRTIDataset): every item also carries its forecast interval in
        # hours, a function of (seed, index) only so that every rank sharing a sample agrees on it
        self.intervals = tuple(intervals) if intervals else None
        self._cache: dict[int, tuple[torch.Tensor, torch.Tensor]] = {}

    def __len__(self):
        return self.length

    def __getitem__(self, idx: int):
        k = idx % self.pool          # a small pool of distinct samples keeps host generation off the critical path
        if k not in self._cache:
            g = torch.Generator().manual_seed(self.seed * 1_000_003 + k * 1009 + self.rank_id)
            shape_c = (self.hb, self.wb, self.cc) if self.channels_last else (self.cc, self.hb, self.wb)
            shape_t = (self.hb, self.wb, self.ct) if self.channels_last else (self.ct, self.hb, self.wb)
            self._cache[k] = (torch.randn(shape_c, generator=g), torch.randn(shape_t, generator=g))
        if self.intervals:
            pick = (self.seed * 7919 + idx * 104729) % len(self.intervals)
            return (*self._cache[k], torch.tensor([float(self.intervals[pick])]))
        return self._cache[k]
