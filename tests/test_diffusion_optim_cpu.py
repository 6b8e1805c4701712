"""TrigFlow objective and sampler, LR / EMA schedules and the flat AdamW optimizer, each against its closed form or
``torch.optim.AdamW`` (reference: parallel_engine.py:21-33, 799-887, 990-997; pp_generate.py:113-119, 228-241, 298-322)."""
import math

import pytest
import torch

from aeris_gb_b200.diffusion import trigflow as TF
from aeris_gb_b200.engine.optim import FlatOptimizer, OptimConfig, ema_beta_at, lr_at, no_decay_names


# ------------------------------------------------------------------------------------------------------ TrigFlow
def test_noise_levels_are_log_uniform_in_sigma():
    g = torch.Generator().manual_seed(0)
    t = TF.sample_noise_level(20000, 0.2, 500.0, 1.0, generator=g)
    tau = torch.tan(t)
    assert 0.2 * 0.999 <= tau.min() and tau.max() <= 500.0 * 1.001
    # the median of a log-uniform law is the geometric mean of its ends
    assert torch.log(tau).median().item() == pytest.approx(0.5 * (math.log(0.2) + math.log(500.0)), abs=0.08)
    u = TF.sample_noise_level(1000, 0.2, 500.0, 1.0, generator=g, law="uniform")
    assert 0 <= u.min() and u.max() <= math.pi / 2


def test_forward_process_target_and_loss_identities():
    g = torch.Generator().manual_seed(1)
    x, z, c = torch.randn(2, 6, 3, generator=g), torch.randn(2, 6, 3, generator=g) * 2.0, torch.randn(2, 6, 4, generator=g)
    t = torch.tensor([0.3, 1.2])
    mi = TF.noise_inputs(x, c, z, t, sigma_data=2.0)
    ct, st = torch.cos(t).view(2, 1, 1), torch.sin(t).view(2, 1, 1)
    assert torch.allclose(mi[..., :3], (ct * x + st * z) / 2.0) and torch.equal(mi[..., 3:], c)
    v = TF.v_target(x, z, t)
    assert torch.allclose(v, ct * z - st * x)
    # (x_t, v) is (x, z) rotated by t: the rotation is undone exactly
    x_t = ct * x + st * z
    assert torch.allclose(ct * x_t - st * v, x, atol=1e-6) and torch.allclose(st * x_t + ct * v, z, atol=1e-6)
    # a perfect prediction has zero loss; weights enter linearly
    assert TF.trigflow_loss(v / 2.0, x, z, t, 2.0, None, None).item() == pytest.approx(0.0, abs=1e-10)
    w_var = torch.tensor([1.0, 2.0, 3.0])
    base = TF.trigflow_loss(torch.zeros_like(v), x, z, t, 2.0, None, None)
    weighted = TF.trigflow_loss(torch.zeros_like(v), x, z, t, 2.0, torch.full((2, 6, 1), 0.5), w_var)
    assert weighted.item() == pytest.approx(0.5 * ((v ** 2) * w_var).sum(-1).mean().item(), rel=1e-6)
    assert base.item() == pytest.approx((v ** 2).sum(-1).mean().item(), rel=1e-6)


def test_sampler_schedule_runs_from_sigma_max_to_zero():
    ts = TF.sampler_schedule(20, 0.2, 500.0, 1.0)
    assert ts.shape == (21,) and ts[-1] == 0 and torch.all(ts[:-1] > ts[1:])
    assert ts[0].item() == pytest.approx(math.atan(500.0), rel=1e-6) and ts[-2].item() == pytest.approx(math.atan(0.2), rel=1e-6)


def test_sampler_integrates_the_exact_flow_of_a_point_mass():
    """Data concentrated in x0: the exact network output is F = (cos t x_t - x0) / (sin t sigma_d); the probability
    flow is then the rotation x(t) = cos t x0 + sin t z, which the sampler must follow down to x0, Heun closer than Euler."""
    g = torch.Generator().manual_seed(2)
    x0 = torch.randn(1, 5, 3, generator=g)
    sd = 1.5

    def denoise(model_in, t):
        x_t = model_in[..., :3] * sd
        tt = t.view(-1, 1, 1)
        return (torch.cos(tt) * x_t - x0) / (torch.sin(tt) * sd)
    cond = torch.zeros(1, 5, 0)
    z = torch.randn(1, 5, 3, generator=g) * sd
    t0 = math.atan(80.0 / sd)
    x_init = math.cos(t0) * x0 + math.sin(t0) * z
    err = {}
    for heun in (False, True):
        y = TF.sample(denoise, cond, x0.shape, 12, 0.02, 80.0, sd, heun=heun, x_init=x_init.clone())
        err[heun] = (y - x0).abs().max().item()
    assert err[True] < 2e-2 and err[True] < err[False]


def test_churn_rotates_toward_fresh_noise():
    g = torch.Generator().manual_seed(3)
    x = torch.randn(4, 7)
    same, s = TF.churn_form2(x, 0.9, 0.0, 1.0)
    assert same is x and s == 0.9
    y, s_hat = TF.churn_form2(x, 0.9, 0.3, 2.0, torch.Generator().manual_seed(5), s_noise=1.003)
    assert s_hat == pytest.approx(math.atan(math.tan(0.9) * 1.3))
    s_l = math.atan(math.tan(s_hat) - math.tan(0.9))
    eps = torch.randn(x.shape, generator=torch.Generator().manual_seed(5)) * 2.0
    assert torch.allclose(y, math.cos(s_l) * x + math.sin(s_l) * 1.003 * eps, atol=1e-6)


def test_latitude_and_variable_weights():
    w = TF.latitude_weights(720, 0.01)
    assert w.shape == (720,) and w.min() > 0 and w.mean().item() == pytest.approx(1.0, abs=2e-3)
    assert w[359].item() > w[0].item() and w[0].item() == pytest.approx(w[-2].item(), rel=0.02)   # equator > poles
    assert TF.latitude_weights(16, 0.0).shape == (16,)
    assert TF.variable_weights(70).shape == (70,) and TF.variable_weights(69).shape == (69,)
    assert TF.variable_weights(6).sum().item() == pytest.approx(1.0)


# ------------------------------------------------------------------------------------------------------ schedules
def test_learning_rate_schedule_pieces():
    c = OptimConfig(lr=1e-3, total_img=1000, lr_rampup_img=100, lr_min_factor=0.1, lr_rampdown_start=2000,
                    lr_rampdown_length=400)
    assert lr_at(0, c.lr, c) == pytest.approx(1e-4)                       # warm-up starts at the floor
    assert lr_at(50, c.lr, c) == pytest.approx(1e-4 + 0.5 * 9e-4)
    assert lr_at(100, c.lr, c) == pytest.approx(1e-3)                     # cosine starts at the base rate
    assert lr_at(550, c.lr, c) == pytest.approx(1e-4 + 0.5 * 9e-4)        # half way down the cosine
    assert lr_at(1000, c.lr, c) == pytest.approx(1e-4) and lr_at(1500, c.lr, c) == pytest.approx(1e-4)
    assert lr_at(2200, c.lr, c) == pytest.approx(1e-4 + 9e-4 * 0.5)       # linear ramp-down window
    assert lr_at(2401, c.lr, c) == pytest.approx(1e-4)


def test_ema_coefficient_follows_the_half_life_with_ramp_up():
    c = OptimConfig(ema_halflife_img=1000, ema_rampup_ratio=0.05, lr_rampdown_start=10 ** 9, lr_rampdown_length=10)
    assert ema_beta_at(100_000, 10, c) == pytest.approx(0.5 ** (10 / 1000))          # steady state
    assert ema_beta_at(2000, 10, c) == pytest.approx(0.5 ** (10 / 100))              # early: half-life = 5 % of images
    assert ema_beta_at(0, 10, c) == pytest.approx(0.0, abs=1e-12)                    # the first update copies the weights
    assert ema_beta_at(10 ** 9 + 11, 10, c) is None                                  # frozen after the ramp-down


def test_weight_decay_groups():
    m = torch.nn.ModuleDict({"proj": torch.nn.Linear(3, 3), "head": torch.nn.Linear(3, 2, bias=False),
                             "norm": torch.nn.LayerNorm(3), "modulation": torch.nn.Linear(3, 3), "w1": torch.nn.Linear(3, 3)})
    names = {n for n, _ in m.named_parameters()}
    assert no_decay_names(m, "custom_decay5") == names and no_decay_names(m, "all") == set()
    nd = no_decay_names(m, "custom_decay")
    assert {"proj.weight", "proj.bias", "head.weight", "norm.weight", "norm.bias"} <= nd
    assert "w1.weight" not in nd and "modulation.weight" not in nd


# ------------------------------------------------------------------------------------------------------ optimizer
def _two_models():
    torch.manual_seed(0)
    a = torch.nn.Sequential(torch.nn.Linear(5, 7), torch.nn.Tanh(), torch.nn.Linear(7, 3))
    b = torch.nn.Sequential(torch.nn.Linear(5, 7), torch.nn.Tanh(), torch.nn.Linear(7, 3))
    b.load_state_dict(a.state_dict())
    return a, b


def test_flat_optimizer_steps_like_torch_adamw_and_tracks_the_ema():
    a, b = _two_models()
    c = OptimConfig(lr=3e-3, betas=(0.85, 0.9), eps=1e-8, weight_decay=0.2, decay_policy="all", grad_clip=False,
                    lr_rampup_img=0, total_img=10 ** 12, lr_min_factor=1.0, ema_halflife_img=50, ema_rampup_ratio=None)
    opt = FlatOptimizer(a, c)
    ref = torch.optim.AdamW(b.parameters(), lr=3e-3, betas=(0.85, 0.9), eps=1e-8, weight_decay=0.2)
    ema = [p.detach().clone() for p in b.parameters()]
    g = torch.Generator().manual_seed(1)
    for _ in range(4):
        x = torch.randn(6, 5, generator=g)
        a(x).pow(2).sum().backward()
        b(x).pow(2).sum().backward()
        opt.step(batch_img=8, grad_scale=0.5)                  # the accumulated gradient is scaled by 1 / (DP GAS)
        for p in b.parameters():
            p.grad.mul_(0.5)
        ref.step()
        ref.zero_grad()
        beta = 0.5 ** (8 / 50)
        for e, p in zip(ema, b.parameters()):
            e.copy_(p.detach().lerp(e, beta))
    for p, q in zip(a.parameters(), b.parameters()):
        assert torch.allclose(p, q, atol=1e-6, rtol=1e-5)
        assert p.grad is None and float(p.main_grad.abs().max()) == 0.0      # folded into the flat buffer, then zeroed
    for (n, e), r in zip(opt.ema_state_dict().items(), ema):
        assert torch.allclose(e, r, atol=1e-6, rtol=1e-5), n
    assert opt.cur_nimg == 32 and opt.step_count == 4


def test_flat_optimizer_clips_by_the_global_norm_and_survives_nans():
    a, b = _two_models()
    c = OptimConfig(lr=1e-2, weight_decay=0.0, decay_policy="all", grad_clip=True, grad_clip_max_norm=0.1,
                    lr_rampup_img=0, lr_min_factor=1.0, use_ema=False)
    opt = FlatOptimizer(a, c)
    x = torch.randn(6, 5, generator=torch.Generator().manual_seed(2))
    a(x).pow(2).sum().backward()
    b(x).pow(2).sum().backward()
    nsq = opt.grad_norm_sq(1.0)
    total = torch.sqrt(sum(p.grad.pow(2).sum() for p in b.parameters()))
    assert float(nsq.sqrt()) == pytest.approx(float(total), rel=1e-5) and float(total) > 0.1
    before = [p.detach().clone() for p in a.parameters()]
    opt.step(batch_img=1, grad_scale=1.0, norm_sq=nsq)
    # Adam's first step moves every weight by lr * sign(g) whatever the clip factor; a clipped, finite update it is
    for p, q in zip(a.parameters(), before):
        assert torch.isfinite(p).all() and float((p.detach() - q).abs().max()) <= 1e-2 * 1.0001
    for p in a.parameters():
        p.main_grad.fill_(float("nan"))
    opt.step(batch_img=1, grad_scale=1.0, norm_sq=torch.tensor([1.0], dtype=torch.float64))
    assert all(torch.isfinite(p).all() for p in a.parameters())          # NaN gradients are zeroed, not applied


# ------------------------------------------------------------------------------------------------------ rollout
def test_autoregressive_rollout_standardises_the_condition_and_adds_the_unstandardised_residual():
    """A stand-in network that knows the residual exactly: y* = 0.1 * (standardised state) + (forcing channel). The
    forecaster must feed it the standardised state and forcing, integrate to y*, and advance the physical state by
    ``y* * t_std + t_mean`` (pp_generate.py:325-333), step after step."""
    from aeris_gb_b200.diffusion.rollout import Forecaster, SamplerConfig
    C, sd = 3, 1.0
    stats = {"x_mean": torch.tensor([1.0, -2.0, 0.5]), "x_std": torch.tensor([2.0, 0.5, 1.5]),
             "t_mean": torch.tensor([0.1, 0.0, -0.2]), "t_std": torch.tensor([0.3, 0.2, 0.1])}
    seen = []

    def denoise(model_in, t):
        x_t, cond_state, forcing = model_in[..., :C] * sd, model_in[..., C:2 * C], model_in[..., 2 * C:]
        seen.append((cond_state.clone(), forcing.clone()))
        y_star = 0.1 * cond_state + forcing
        tt = t.view(-1, 1, 1)
        return (torch.cos(tt) * x_t - y_star) / (torch.sin(tt) * sd)
    fc = Forecaster(denoise, stats, SamplerConfig(n_steps=16, sigma_min=0.02, sigma_max=80.0, sigma_data=sd), C)
    assert fc.model_evals_per_forecast_step() == 31
    g = torch.Generator().manual_seed(0)
    state = torch.randn(2, 4, C, generator=g) * 3.0
    forc = [torch.randn(2, 4, 1, generator=g).expand(2, 4, C).contiguous() for _ in range(2)]
    steps = []
    final = fc.rollout(state, lambda k: forc[k], 2, generator=g, on_step=lambda k, s: steps.append((k, s.clone())))
    expect = state
    for k in range(2):
        cond = (expect - stats["x_mean"]) / stats["x_std"]
        expect = expect + (0.1 * cond + forc[k]) * stats["t_std"] + stats["t_mean"]
        assert torch.allclose(steps[k][1], expect, atol=5e-3), k
    assert [k for k, _ in steps] == [0, 1] and torch.equal(final, steps[-1][1])
    assert torch.allclose(seen[0][0], (state - stats["x_mean"]) / stats["x_std"], atol=1e-6)
    assert torch.equal(seen[0][1], forc[0])
