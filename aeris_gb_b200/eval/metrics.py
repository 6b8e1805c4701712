"""Ensemble forecast scores, accumulated on the device: latitude-weighted MSE of member 0 and of the ensemble mean, the
fair CRPS ``E|X - y| - sum_ij |X_i - X_j| / (2 N (N-1))`` and the spread/skill ratio.

Reference: src/aeris/pp_generate.py:346-398 (per rollout step, per channel; five all-reduces with sleeps in between,
results accumulated in ``err[steps, 5, C]``) and :486-496 (``*_err_aggregate.npy`` = raw sums, ``*_err.npy`` =
``[steps, 4, C]`` with RMSE(first), RMSE(mean), CRPS, spread/skill). Here the five partial sums travel in ONE packed
all-reduce, and nothing leaves the device until :meth:`finalize`.
"""
from __future__ import annotations

import numpy as np
import torch
import torch.distributed as dist

HEADLINE = {"t2m": "2m_temperature", "u10m": "10m_u_component_of_wind", "v10m": "10m_v_component_of_wind",
            "mslp": "mean_sea_level_pressure", "z500": "geopotential_500", "t850": "temperature_850",
            "q700": "specific_humidity_700", "u850": "u_component_of_wind_850", "v850": "v_component_of_wind_850"}


def step_sums(members: torch.Tensor, label: torch.Tensor, w_lat: torch.Tensor) -> torch.Tensor:
    """members [M, C, h, w] (this rank's block, physical units), label [C, h, w], w_lat [h] -> [5, C] partial sums over
    this block: (w (y - x0)^2, w (y - mean)^2, w mean_m |x - y|, w sum_ij |xi - xj| / (2 M (M-1)), w var_m)."""
    M = members.shape[0]
    w = w_lat.view(1, -1, 1)
    e1 = (w * (label - members[0]) ** 2).sum(dim=(-1, -2))
    em = (w * (label - members.mean(dim=0)) ** 2).sum(dim=(-1, -2))
    ca = (w.unsqueeze(0) * (members - label.unsqueeze(0)).abs()).sum(dim=(0, 2, 3)) / M
    if M > 1:
        # sum_ij |xi - xj| through sorting: for sorted values, sum_ij |xi - xj| = 2 * sum_k (2k - M + 1) x_(k)
        srt, _ = members.sort(dim=0)
        coef = (2 * torch.arange(M, device=members.device, dtype=members.dtype) - M + 1).view(M, 1, 1, 1)
        pair = 2 * (coef * srt).sum(dim=0)
        cs = (w * pair).sum(dim=(-1, -2)) / (2 * M * (M - 1))
        var = (w * members.var(dim=0)).sum(dim=(-1, -2))
    else:
        cs = torch.zeros_like(e1)
        var = torch.zeros_like(e1)
    return torch.stack([e1, em, ca, cs, var])


class EnsembleMetrics:
    def __init__(self, rollout_steps: int, n_channels: int, n_pixels: int, device, group=None):
        self.err = torch.zeros((rollout_steps, 5, n_channels), device=device, dtype=torch.float64)
        self.n_pixels, self.group, self.count = n_pixels, group, 0

    def update(self, step: int, members: torch.Tensor, label: torch.Tensor, w_lat: torch.Tensor):
        s = step_sums(members.double(), label.double(), w_lat.double())
        if self.group is not None and dist.is_initialized() and dist.get_world_size(self.group) > 1:
            dist.all_reduce(s, group=self.group)                      # one packed reduction over the WP ranks
        s = s / self.n_pixels
        s[4] = s[4].sqrt()
        self.err[step] += s

    def end_initial_condition(self):
        self.count += 1

    def running_line(self, step: int, channel: int, interval: int = 6) -> str:
        """Scores of one channel at one lead time over the initial conditions seen so far, the current one included
        (the reference prints this for 2 m temperature after every rollout step, pp_generate.py:461-468)."""
        e = (self.err[step, :, channel] / (self.count + 1)).tolist()
        rmse_mean = max(e[1], 0.0) ** 0.5
        return (f"{interval * (step + 1)}h scores at ic {self.count + 1}: {max(e[0], 0.0) ** 0.5:.4f}, {rmse_mean:.4f}, "
                f"{e[2] - e[3]:.4f}, {e[4] / max(rmse_mean, 1e-30):.4f}")

    def finalize(self) -> tuple[np.ndarray, np.ndarray]:
        """(aggregate [steps, 5, C] raw sums, scores [steps, 4, C] = RMSE first, RMSE mean, CRPS, spread/skill)."""
        n = max(self.count, 1)
        e = self.err / n
        out = torch.stack([e[:, 0].sqrt(), e[:, 1].sqrt(), e[:, 2] - e[:, 3], e[:, 4] / e[:, 1].sqrt().clamp_min(1e-30)],
                          dim=1)
        return self.err.cpu().numpy(), out.cpu().numpy()

    def headline_table(self, variables: list[str], steps=(0, 1, 3), interval: int = 6) -> str:
        _, sc = self.finalize()
        lines = []
        for i in steps:
            if i >= sc.shape[0]:
                continue
            lines.append(f"{interval * (i + 1)}h")
            for key, name in HEADLINE.items():
                if name not in variables:
                    continue
                j = variables.index(name)
                k = 1000.0 if key == "q700" else 1.0
                lines.append(f"{key:>5}: {sc[i, 0, j] * k:.4f}, {sc[i, 1, j] * k:.4f}, {sc[i, 2, j] * k:.4f}, {sc[i, 3, j]:.4f}")
        return "\n".join(lines)
