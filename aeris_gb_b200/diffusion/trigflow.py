"""TrigFlow v-prediction: noise draw, forward process, training loss, sampler schedule and Euler/Heun updates.

Reference: noise draw src/aeris/parallelism/parallel_engine.py:21-33; forward process :673-678; loss :990-997 with the
latitude weights of :635-639 and the hard-coded per-variable weights of :966-989; sampler schedule
src/aeris/pp_generate.py:113-119; Euler/Heun update :298-322; churn (form 2) :228-241.
"""
from __future__ import annotations

import math

import torch

# Per-variable loss weights of the published 70-channel configuration (parallel_engine.py:966-973): 2 m temperature,
# three other surface fields, 5 variables x 13 pressure levels (weights proportional to pressure), sea-surface temp.
_LEVEL_W = [0.0013, 0.0026, 0.0039, 0.0052, 0.0065, 0.0078, 0.0104, 0.0130, 0.0156, 0.0182, 0.0220, 0.0240, 0.0259]
W_VAR_70 = [0.1562, 0.0156, 0.0156, 0.0156] + _LEVEL_W * 5 + [0.0156]
_LEVEL_W69 = [0.00131726, 0.00263453, 0.00395179, 0.00526905, 0.00658631, 0.00790358, 0.0105381, 0.01317263,
              0.01580715, 0.01844168, 0.02239347, 0.02436936, 0.02634525]
W_VAR_69 = [0.15873015, 0.01587301, 0.01587301, 0.01587301] + _LEVEL_W69 * 5


def variable_weights(n_channels: int, device=None) -> torch.Tensor:
    if n_channels == 70:
        w = W_VAR_70
    elif n_channels == 69:
        w = W_VAR_69
    else:
        w = [1.0 / n_channels] * n_channels
    return torch.tensor(w, dtype=torch.float32, device=device)


def latitude_weights(n_lat: int, w_lat_add: float = 0.0, drop_first_row: bool | None = None) -> torch.Tensor:
    """``(cos(lat) + w_lat_add) / mean`` per image row. For the 720-row grid the reference evaluates 721 rows from
    -90 to 90 degrees, normalises by their mean and drops the first row (parallel_engine.py:536,636-637)."""
    if drop_first_row is None:
        drop_first_row = n_lat == 720
    n = n_lat + 1 if drop_first_row else n_lat
    w = torch.cos(torch.deg2rad(torch.linspace(-90, 90, n))) + w_lat_add
    w = w / w.mean()
    return w[1:] if drop_first_row else w


def sample_noise_level(batch: int, sigma_min: float, sigma_max: float, sigma_data: float, generator=None,
                       device=None, law: str = "loguniform") -> torch.Tensor:
    """t in [0, pi/2]. ``loguniform``: tau ~ LogUniform[sigma_min, sigma_max], t = atan(tau / sigma_data)
    (parallel_engine.py:22-30); ``uniform``: t ~ U(0, pi/2)."""
    u = torch.rand(batch, generator=generator, device=device)
    if law == "uniform":
        return u * (math.pi / 2)
    ls = math.log(sigma_min) + u * (math.log(sigma_max) - math.log(sigma_min))
    return torch.atan(torch.exp(ls) / sigma_data)


def _bcast(t: torch.Tensor, like: torch.Tensor) -> torch.Tensor:
    return t.view(-1, *([1] * (like.dim() - 1)))


def noise_inputs(x: torch.Tensor, cond: torch.Tensor, z: torch.Tensor, t: torch.Tensor, sigma_data: float):
    """Model input ``cat([x_t / sigma_d, cond])`` with ``x_t = cos t * x + sin t * z`` (z already scaled by sigma_d).
    x, z: [B, ..., C]; cond: [B, ..., Cc]; t: [B]."""
    ct, st = _bcast(torch.cos(t), x), _bcast(torch.sin(t), x)
    x_t = ct * x + st * z
    return torch.cat([x_t / sigma_data, cond], dim=-1)


def v_target(x: torch.Tensor, z: torch.Tensor, t: torch.Tensor) -> torch.Tensor:
    return _bcast(torch.cos(t), x) * z - _bcast(torch.sin(t), x) * x


def trigflow_loss(pred: torch.Tensor, x: torch.Tensor, z: torch.Tensor, t: torch.Tensor, sigma_data: float,
                  w_lat: torch.Tensor | None, w_var: torch.Tensor | None) -> torch.Tensor:
    """``mean_tokens sum_c w_lat * w_var * (sigma_d * F - v_t)^2`` (parallel_engine.py:995-997). ``w_lat`` broadcasts
    against pred[..., :1] (per token), ``w_var`` against the channel axis."""
    err = (sigma_data * pred - v_target(x, z, t)) ** 2
    if w_var is not None:
        err = err * w_var
    if w_lat is not None:
        err = err * w_lat
    return err.sum(dim=-1).mean()


def sampler_schedule(n_steps: int, sigma_min: float, sigma_max: float, sigma_data: float, rho: float = 10.0,
                     device=None) -> torch.Tensor:
    """t_i = atan(sigma_i / sigma_d), sigma_i = (smax^(1/rho) + i/(N-1) (smin^(1/rho) - smax^(1/rho)))^rho, then 0
    appended (pp_generate.py:113-119). Returns N+1 values, decreasing."""
    i = torch.arange(n_steps, dtype=torch.float64, device=device)
    denom = max(n_steps - 1, 1)
    sig = (sigma_max ** (1 / rho) + i / denom * (sigma_min ** (1 / rho) - sigma_max ** (1 / rho))) ** rho
    t = torch.atan(sig / sigma_data)
    return torch.cat([t, torch.zeros(1, dtype=t.dtype, device=device)]).float()


def churn_form2(x_t: torch.Tensor, s_cur: float, gamma: float, sigma_data: float, generator=None,
                s_noise: float = 1.0):
    """Raise the noise level from s_cur to s_hat = atan(tan(s_cur) * (1 + gamma)) by rotating x_t toward fresh noise
    (pp_generate.py:228-241, 'form 2'): s_l = atan(tan s_hat - tan s_cur), x <- cos(s_l) x + sin(s_l) sigma_d eps,
    a pure rotation in the (signal, noise) plane; ``s_noise`` scales the fresh noise (the reference's ``S_noise``)."""
    if gamma <= 0:
        return x_t, s_cur
    s_hat = math.atan(math.tan(s_cur) * (1 + gamma))
    s_l = math.atan(max(math.tan(s_hat) - math.tan(s_cur), 0.0))
    eps = torch.randn(x_t.shape, generator=generator, device=x_t.device, dtype=x_t.dtype) * sigma_data
    return math.cos(s_l) * x_t + math.sin(s_l) * s_noise * eps, s_hat


@torch.no_grad()
def sample(denoise, cond: torch.Tensor, shape, n_steps: int, sigma_min: float, sigma_max: float, sigma_data: float,
           rho: float = 10.0, heun: bool = True, generator=None, s_churn: float = 0.0, s_min: float = 0.0,
           s_max: float = float("inf"), x_init: torch.Tensor | None = None, s_noise: float = 1.0) -> torch.Tensor:
    """Deterministic TrigFlow sampler: Euler steps with a 2nd-order Heun correction on all but the last step
    (pp_generate.py:298-322). ``denoise(model_in [B,...,C+Cc], t [B]) -> F`` is the network.
    Returns the sample at t = 0 (same shape as ``shape``)."""
    device = cond.device
    ts = sampler_schedule(n_steps, sigma_min, sigma_max, sigma_data, rho, device=device)
    x = x_init if x_init is not None else torch.randn(shape, generator=generator, device=device) * sigma_data
    B = x.shape[0]
    for i in range(n_steps):
        s, tn = float(ts[i]), float(ts[i + 1])
        if s_churn > 0:
            gamma = min(s_churn / n_steps, math.sqrt(2) - 1) if s_min <= math.tan(s) * sigma_data <= s_max else 0.0
            x, s = churn_form2(x, s, gamma, sigma_data, generator, s_noise)
        d = tn - s
        f_s = denoise(torch.cat([x / sigma_data, cond], dim=-1), torch.full((B,), s, device=device))
        x_e = x + d * sigma_data * f_s
        if heun and i < n_steps - 1:
            f_t = denoise(torch.cat([x_e / sigma_data, cond], dim=-1), torch.full((B,), tn, device=device))
            x = x + d * sigma_data * 0.5 * (f_s + f_t)
        else:
            x = x_e
    return x
