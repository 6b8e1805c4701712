"""Autoregressive ensemble rollout, resident on the device.

Each forecast step draws the standardised residual with the TrigFlow sampler and adds it to the state:
``X_{k+1} = X_k + unstandardize_t(Y)``, ``condition = standardize_x(X_{k+1})`` with the forcing channels
(radiation at T, surface geopotential, land-sea mask, radiation at T+1) appended from data.
Reference: src/aeris/pp_generate.py:159-333 and src/aeris_wp_inference/inference.py:101-186, which move the state to
the host and through numpy for every (un)standardisation; here the state never leaves the GPU.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from . import trigflow as TF


@dataclass
class SamplerConfig:
    n_steps: int = 20
    sigma_min: float = 0.2
    sigma_max: float = 500.0
    sigma_data: float = 1.0
    rho: float = 10.0
    heun: bool = True
    s_churn: float = 0.0
    s_min: float = 0.0
    s_max: float = float("inf")


class Forecaster:
    """``denoise(model_in [M, ..., C_in], t [M]) -> F [M, ..., C_out]`` is any callable (a model on one GPU, a
    window-parallel model on this rank's block, or a pipeline engine)."""

    def __init__(self, denoise, stats: dict[str, torch.Tensor], sampler: SamplerConfig, out_channels: int):
        self.denoise, self.stats, self.s, self.C = denoise, stats, sampler, out_channels

    def std_x(self, x):
        return (x - self.stats["x_mean"][:x.shape[-1]]) / self.stats["x_std"][:x.shape[-1]]

    def unstd_t(self, y):
        return y * self.stats["t_std"][:y.shape[-1]] + self.stats["t_mean"][:y.shape[-1]]

    @torch.no_grad()
    def step(self, state: torch.Tensor, forcing: torch.Tensor | None, generator=None) -> torch.Tensor:
        """state [M, ..., C_out] in physical units; forcing [M, ..., C_f] already standardised. Returns the next
        state."""
        cond = self.std_x(state)
        if forcing is not None:
            cond = torch.cat([cond, forcing], dim=-1)
        s = self.s
        y = TF.sample(self.denoise, cond, state.shape, s.n_steps, s.sigma_min, s.sigma_max, s.sigma_data, s.rho,
                      heun=s.heun, generator=generator, s_churn=s.s_churn, s_min=s.s_min, s_max=s.s_max)
        return state + self.unstd_t(y)

    @torch.no_grad()
    def rollout(self, state0: torch.Tensor, forcings, n_rollout: int, generator=None, on_step=None) -> torch.Tensor:
        """``forcings(k)`` -> standardised forcing for step k (or None). ``on_step(k, state)`` is called after every
        step (metrics, output writers). Returns the final state."""
        x = state0
        for k in range(n_rollout):
            x = self.step(x, forcings(k) if forcings is not None else None, generator)
            if on_step is not None:
                on_step(k, x)
        return x

    def model_evals_per_forecast_step(self) -> int:
        return 2 * self.s.n_steps - 1 if self.s.heun else self.s.n_steps
