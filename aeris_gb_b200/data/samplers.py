"""Samplers: endless rank-strided sampler with windowed shuffling, and a Subset that forwards attributes.

Reference: ``InfiniteSampler`` src/aeris/data/samplers.py:14-47 (a variant of the EDM sampler: a permutation that is
re-shuffled locally inside a sliding window as it is consumed), ``AttributeSubset`` :55-62.
"""
from __future__ import annotations

import numpy as np
import torch
from torch.utils.data import Sampler, Subset


class InfiniteSampler(Sampler):
    def __init__(self, dataset, rank: int = 0, num_replicas: int = 1, shuffle: bool = True, seed: int = 0,
                 window_size: float = 0.5, start_idx: int = 0):
        assert len(dataset) > 0 and num_replicas > 0 and 0 <= rank < num_replicas and 0 <= window_size <= 1
        self.n, self.rank, self.num_replicas = len(dataset), rank, num_replicas
        self.shuffle, self.seed, self.window_size, self.start_idx = shuffle, seed, window_size, start_idx

    def __iter__(self):
        order = np.arange(self.n)
        rnd, window = None, 0
        if self.shuffle:
            rnd = np.random.default_rng(self.seed)     # the generator class fixes the sample order for a seed
            rnd.shuffle(order)
            window = int(np.rint(order.size * self.window_size))
        idx = self.start_idx
        while True:
            i = idx % order.size
            if idx % self.num_replicas == self.rank:
                yield int(order[i])
            if window >= 2:
                j = (i - rnd.integers(window)) % order.size
                order[i], order[j] = order[j], order[i]
            idx += 1


class AttributeSubset(Subset):
    """``Subset`` whose unknown attributes fall through to the wrapped dataset."""

    def __getattr__(self, name):
        return getattr(self.dataset, name)
