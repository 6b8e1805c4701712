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
    s_noise: float = 1.0            # scale of the fresh noise that the churn mixes in


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
    def step(self, state: torch.Tensor, forcing: torch.Tensor | None, generator=None,
             x_init: torch.Tensor | None = None) -> torch.Tensor:
        """state [M, ..., C_out] in physical units; forcing [M, ..., C_f] already standardised. Returns the next
        state. ``x_init`` replaces the sampler's initial noise draw."""
        cond = self.std_x(state)
        if forcing is not None:
            cond = torch.cat([cond, forcing], dim=-1)
        s = self.s
        y = TF.sample(self.denoise, cond, state.shape, s.n_steps, s.sigma_min, s.sigma_max, s.sigma_data, s.rho,
                      heun=s.heun, generator=generator, s_churn=s.s_churn, s_min=s.s_min, s_max=s.s_max,
                      x_init=x_init, s_noise=s.s_noise)
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


class DeviceForecaster(Forecaster):
    """The same rollout with every sampler-side operation on this library's CUDA kernels: standardisation, initial
    noise and churn from the counter-based generator, window partition + position encoding + input projection, the
    fp32 output head, Euler/Heun updates written back in image order, un-standardisation + residual add. The state is
    this rank's image block ``[M, hb, wb, C_out]`` and never leaves the device (the reference moves it through host
    numpy at every step, src/aeris/pp_generate.py:327-333).

    ``model`` is an :class:`AerisModel` on a CUDA device, ``ctx`` its :class:`StreamContext` for ``M`` members;
    ``member0`` is the global index of this rank's first member (distinct members draw distinct noise; the ranks of one
    window-parallel group pass the same value and draw consistent noise for their blocks)."""

    def __init__(self, model, ctx, stats, sampler: SamplerConfig, out_channels: int, seed: int = 0, member0: int = 0):
        super().__init__(None, stats, sampler, out_channels)
        from ..models import fused_io
        self.model, self.ctx, self.member0 = model, ctx, member0
        self.seed, self.draws = seed, 0
        dev = next(model.parameters()).device
        self.ape = fused_io.ape_tables(model.cfg, dev)
        xs, xm = stats["x_std"][:out_channels].float(), stats["x_mean"][:out_channels].float()
        self._std_a, self._std_b = (1.0 / xs).contiguous(), (-xm / xs).contiguous()
        self._un_a = stats["t_std"][:out_channels].float().contiguous()
        self._un_b = stats["t_mean"][:out_channels].float().contiguous()

    def _next_seed(self) -> int:
        self.draws += 1
        return (self.seed << 32) + self.draws

    @torch.no_grad()
    def step(self, state: torch.Tensor, forcing: torch.Tensor | None, generator=None, x_init=None) -> torch.Tensor:
        import math
        from ..models import fused_io
        from ..ops import diffusion as DF
        s = self.s
        M = state.shape[0]
        state = state.contiguous()
        geom = DF.make_geom(self.ctx.grid, M, self.ctx.rank, self.member0)
        cond = DF.affine_channels(state, self._std_a, self._std_b)
        c_img = torch.cat([cond, forcing], dim=-1).contiguous() if forcing is not None else cond
        plan = fused_io.IoPlan(geom, s.sigma_data, 0, False, self.ape[0], self.ape[1])
        ts = TF.sampler_schedule(s.n_steps, s.sigma_min, s.sigma_max, s.sigma_data, s.rho).tolist()
        if x_init is not None:
            x = x_init.clone()
        else:
            x = DF.noise_mix(torch.empty_like(state), 0.0, s.sigma_data, self._next_seed(), geom)
        x_e = torch.empty_like(x)
        level = lambda v: torch.full((M,), v, device=state.device)
        for i in range(s.n_steps):
            cur, nxt = ts[i], ts[i + 1]
            if s.s_churn > 0 and s.s_min <= math.tan(cur) * s.sigma_data <= s.s_max:
                gamma = min(s.s_churn / s.n_steps, math.sqrt(2) - 1)
                hat = math.atan(math.tan(cur) * (1 + gamma))
                rot = math.atan(max(math.tan(hat) - math.tan(cur), 0.0))
                DF.noise_mix(x, math.cos(rot), math.sin(rot) * s.sigma_data * s.s_noise, self._next_seed(), geom)
                cur = hat
            d = (nxt - cur) * s.sigma_data
            f_s = self.model.predict_images(x, c_img, level(cur), self.ctx, plan)
            DF.sampler_update(x_e, x, f_s, None, d, 0.0, geom)
            if s.heun and i < s.n_steps - 1:
                f_t = self.model.predict_images(x_e, c_img, level(nxt), self.ctx, plan)
                DF.sampler_update(x, x, f_s, f_t, 0.5 * d, 0.5 * d, geom)
            else:
                x, x_e = x_e, x
        return DF.affine_channels(x, self._un_a, self._un_b, add=state)
