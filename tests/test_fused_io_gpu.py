"""Noising / embedding / output head / loss / sampler kernels against plain PyTorch fp32 formulations."""
import math

import pytest
import torch

from conftest import rel_err

pytestmark = pytest.mark.gpu


def _cfg(wp=(1, 1), sp=1):
    from aeris_gb_b200.models.aeris import AerisConfig
    return AerisConfig(img=(32, 64), window=(8, 8), in_channels=20, out_channels=6, dim=256, heads=4, head_dim=64,
                       mlp_dim=512, n_layers=2, sublayers=1, norm_eps=1e-3, chunk_windows=5, wp=wp, sp=sp)


def _noise_image(grid, B, seed, C, rank=0):
    """Unit Gaussian noise of one rank's block, [B, hb, wb, C], straight from the counter-based generator."""
    from aeris_gb_b200.ops import diffusion as DF
    g = DF.make_geom(grid, B, rank)
    z = torch.zeros((B, g.block_shape[1], g.block_shape[2], C), device="cuda")
    return DF.noise_mix(z, 0.0, 1.0, seed, g)


def test_noise_statistics_and_layout_invariance():
    from aeris_gb_b200.models import layout as LY
    full = LY.Grid(32, 64, 8, 8)
    z = _noise_image(full, 3, 77, 6)
    assert abs(z.mean().item()) < 0.02 and abs(z.std().item() - 1.0) < 0.02
    assert abs((z[..., 0] * z[..., 1]).mean().item()) < 0.03          # channels independent
    assert abs((z[:, :, 1:] * z[:, :, :-1]).mean().item()) < 0.03     # neighbouring pixels independent
    assert not torch.equal(z, _noise_image(full, 3, 78, 6))
    # the block of every rank of a 2 x 2 window-parallel grid is the matching slice of the single-rank field
    wp = LY.Grid(32, 64, 8, 8, 2, 2)
    for r in range(4):
        zr = _noise_image(wp, 3, 77, 6, rank=r)
        ry, rx = wp.rank_coords(r)
        assert torch.equal(zr, z[:, ry * 16:(ry + 1) * 16, rx * 32:(rx + 1) * 32])


@pytest.mark.parametrize("sp", [1, 2])
def test_embed_matches_reference(sp):
    from aeris_gb_b200.diffusion import trigflow as TF
    from aeris_gb_b200.models import fused_io, layout as LY
    from aeris_gb_b200.models.aeris import InputStage, StreamContext
    from aeris_gb_b200.ops import diffusion as DF
    torch.manual_seed(0)
    cfg = _cfg(sp=sp)
    grid = cfg.grid()
    B, seed, sd = 2, 5, 1.3
    rank = sp - 1                      # the last sequence slice when sp = 2
    stage = InputStage(cfg).cuda()
    Cx, Cc = cfg.out_channels, cfg.in_channels - cfg.out_channels
    x = torch.randn(B, 32, 64, Cx, device="cuda")
    c = torch.randn(B, 32, 64, Cc, device="cuda")
    t = torch.tensor([0.4, 1.1], device="cuda")
    cs = torch.stack([t.cos(), t.sin()], 1).contiguous()
    ay, ax = fused_io.ape_tables(cfg, "cuda")
    plan = fused_io.IoPlan(DF.make_geom(grid, B, rank), sd, seed, True, ay, ax)
    out = fused_io.EmbedFn.apply(x, c, cs, stage.proj.weight, stage.proj.bias, plan)
    dout = torch.randn_like(out)
    out.backward(dout)
    gw, gb = stage.proj.weight.grad.clone(), stage.proj.bias.grad.clone()
    stage.proj.weight.grad = stage.proj.bias.grad = None
    # reference: same noise, PyTorch fp32
    z = _noise_image(grid, B, seed, Cx, rank) * sd
    tok = lambda img: LY.image_to_tokens(img, grid, (0, 0), rank)
    rows = grid.tokens_per_rank
    model_in = TF.noise_inputs(tok(x), tok(c), tok(z), t.repeat_interleave(rows), sd)
    ctx = StreamContext(cfg, B, rank)
    ref, _ = stage(model_in, t, ctx)          # PyTorch path of the stage (adds the position encoding, projects)
    ref32 = stage.proj(model_in + stage.ape_tokens(ctx, "cuda").repeat(B, 1))
    assert rel_err(out, ref32) < 4e-3
    assert (out.float() - ref32).abs().max() <= 0.02 * ref32.abs().max()
    ref32.backward(dout.float())
    assert rel_err(gw, stage.proj.weight.grad) < 2e-3
    assert rel_err(gb, stage.proj.bias.grad) < 2e-3
    assert rel_err(out, ref) < 8e-3


def test_head_loss_matches_reference():
    from aeris_gb_b200.diffusion import trigflow as TF
    from aeris_gb_b200.models import fused_io, layout as LY
    from aeris_gb_b200.models.aeris import OutputStage
    from aeris_gb_b200.ops import diffusion as DF
    torch.manual_seed(0)
    cfg = _cfg()
    grid = cfg.grid()
    B, seed, sd = 2, 9, 0.8
    stage = OutputStage(cfg).cuda()
    torch.nn.init.normal_(stage.modulation[-1].weight, std=0.05)
    torch.nn.init.normal_(stage.norm.weight, mean=1.0, std=0.1)
    T = B * grid.tokens_per_rank
    xs = torch.randn(T, cfg.dim, device="cuda").bfloat16().requires_grad_(True)
    dt = torch.randn(B, cfg.dim, device="cuda").bfloat16()
    x_img = torch.randn(B, 32, 64, cfg.out_channels, device="cuda")
    t = torch.tensor([0.4, 1.1], device="cuda")
    cs = torch.stack([t.cos(), t.sin()], 1).contiguous()
    w_var = torch.rand(cfg.out_channels, device="cuda") + 0.5
    w_lat = TF.latitude_weights(32, 0.01).cuda()
    plan = fused_io.IoPlan(DF.make_geom(grid, B, 0), sd, seed, True, None, None, w_var, w_lat,
                           cfg.eps(torch.float32))
    params = [p for p in stage.parameters()]
    loss = stage.loss_images(xs, dt, x_img, cs, plan)
    (loss * 1.7).backward()
    got = [xs.grad.clone()] + [p.grad.clone() for p in params]
    xs.grad = None
    for p in params:
        p.grad = None
    # reference
    z = LY.image_to_tokens(_noise_image(grid, B, seed, cfg.out_channels) * sd, grid, (0, 0), 0)
    x_tok = LY.image_to_tokens(x_img, grid, (0, 0), 0)
    rows = grid.tokens_per_rank
    shift, scale = stage.modulation(dt.float()).chunk(2, dim=1)
    xf = xs.float().view(B, rows, -1)
    xn = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + cfg.eps(torch.float32)) * stage.norm.weight
    pred = stage.head(xn * (1 + scale.unsqueeze(1)) + shift.unsqueeze(1)).view(T, -1)
    tr = t.repeat_interleave(rows)
    wl = LY.image_to_tokens(w_lat.view(1, -1, 1, 1).expand(1, 32, 64, 1), grid, (0, 0), 0).repeat(B, 1)
    err = (sd * pred - TF.v_target(x_tok, z, tr)) ** 2 * w_var * wl
    ref = err.sum(-1).view(B, rows).mean(1).sum()
    (ref * 1.7).backward()
    assert abs(loss.item() - ref.item()) < 2e-4 * abs(ref.item())
    want = [xs.grad] + [p.grad for p in params]
    names = ["dx"] + [n for n, _ in stage.named_parameters()]
    for n, a, b in zip(names, got, want):
        assert rel_err(a, b) < 2e-2, (n, rel_err(a, b))
    # forward-only head used by the sampler
    f = stage.predict_tokens(xs.detach(), dt)
    assert f.shape == (T, 128) and rel_err(f[:, :cfg.out_channels], pred) < 1e-4
    assert f[:, cfg.out_channels:].abs().max().item() == 0.0


def test_trainer_fused_io_matches_token_path():
    """Whole model: loss and gradients of the image-layout CUDA path equal the token path fed with the same noise."""
    from aeris_gb_b200.engine.optim import OptimConfig
    from aeris_gb_b200.engine.trainer import DiffusionConfig, Trainer
    cfg = _cfg()
    dcfg = DiffusionConfig(cond_channels=cfg.in_channels - cfg.out_channels, sigma_data=1.0)
    tr = Trainer(cfg, OptimConfig(), dcfg, "cuda", fused_io=True)
    B = 2
    x = torch.randn(B, 32, 64, cfg.out_channels, device="cuda")
    c = torch.randn(B, 32, 64, dcfg.cond_channels, device="cuda")
    t = torch.tensor([0.5, 1.0], device="cuda")
    params = [p for p in tr.model.parameters() if p.requires_grad]
    loss = tr.loss_images(x, c, t, seed=11)
    loss.backward()
    got = [b.clone() for b in tr.opt.grad_buffers()]
    for b in tr.opt.grad_buffers():
        b.zero_()
    z = _noise_image(tr.grid, B, 11, cfg.out_channels) * dcfg.sigma_data
    ref = tr.loss_tokens(tr.block_to_tokens(x), tr.block_to_tokens(c), t, tr.block_to_tokens(z))
    ref.backward()
    assert abs(loss.item() - ref.item()) < 2e-3 * abs(ref.item())
    for a, b in zip(got, tr.opt.grad_buffers()):
        assert rel_err(a, b) < 3e-2, rel_err(a, b)


def test_sampler_affine_gemv():
    from aeris_gb_b200.models import layout as LY
    from aeris_gb_b200.ops import diffusion as DF
    torch.manual_seed(0)
    grid = LY.Grid(32, 64, 8, 8, 1, 2)
    B, C = 2, 6
    g = DF.make_geom(grid, B, 1)
    x = torch.randn(B, 32, 32, C, device="cuda")
    pa = torch.randn(g.rows, 128, device="cuda")
    pb = torch.randn(g.rows, 128, device="cuda")
    out = DF.sampler_update(torch.empty_like(x), x, pa, pb, 0.3, -0.2, g)
    # token order of rank 1 = its block in window-major order
    to_tok = lambda img: img.view(B, 4, 8, 4, 8, C).permute(0, 1, 3, 2, 4, 5).reshape(-1, C)
    ref = to_tok(x) + 0.3 * pa[:, :C] - 0.2 * pb[:, :C]
    assert torch.allclose(to_tok(out), ref, atol=1e-6)
    a, b = torch.rand(C, device="cuda") + 0.5, torch.randn(C, device="cuda")
    assert torch.allclose(DF.affine_channels(x, a, b, add=out), x * a + b + out, atol=1e-6)
    W = torch.randn(300, 256, device="cuda").bfloat16()
    bias = torch.randn(300, device="cuda")
    v = torch.randn(3, 256, device="cuda")
    y = DF.gemv_bias_act(W, bias, v, act=1, silu_in=True)
    ref = torch.nn.functional.silu(torch.nn.functional.silu(v) @ W.float().t() + bias)
    assert rel_err(y, ref) < 1e-4
    y32 = DF.gemv_bias_act(W.float(), None, v)
    assert rel_err(y32, v @ W.float().t()) < 1e-5


@pytest.mark.parametrize("heun,churn", [(True, 0.0), (False, 0.0), (True, 1.0)])
def test_device_forecaster_matches_pytorch_sampler(heun, churn):
    from aeris_gb_b200.diffusion.rollout import DeviceForecaster, Forecaster, SamplerConfig
    from aeris_gb_b200.models.aeris import AerisModel, StreamContext
    torch.manual_seed(3)
    cfg = _cfg()
    grid = cfg.grid()
    model = AerisModel(cfg).cuda().eval()
    torch.nn.init.normal_(model.output_stage.head.weight, std=0.05)
    M, C = 2, cfg.out_channels
    C_f = cfg.in_channels - 2 * C
    ctx = StreamContext(cfg, M)
    stats = {"x_mean": torch.randn(C, device="cuda"), "x_std": torch.rand(C, device="cuda") + 0.5,
             "t_mean": torch.randn(C, device="cuda") * 0.1, "t_std": torch.rand(C, device="cuda") + 0.5}
    sampler = SamplerConfig(n_steps=3, sigma_min=0.2, sigma_max=80.0, sigma_data=1.0, heun=heun, s_churn=churn)
    state = torch.randn(M, 32, 64, C, device="cuda")
    forcing = torch.randn(M, 32, 64, C_f, device="cuda")
    dev_fc = DeviceForecaster(model, ctx, stats, sampler, C, seed=4)
    out = dev_fc.step(state, forcing)
    assert out.shape == state.shape and torch.isfinite(out).all()
    if churn > 0:
        # fresh noise at every churned step: a second call differs, and differs from a churn-free run
        assert not torch.allclose(out, DeviceForecaster(model, ctx, stats, sampler, C, seed=5).step(state, forcing))
        return

    def denoise(model_in, t):
        with torch.no_grad():
            return model(model_in, t)

    z = _noise_image(grid, M, (4 << 32) + 1, C) * sampler.sigma_data
    ref = Forecaster(denoise, stats, sampler, C).step(state, forcing, x_init=z)
    assert rel_err(out - state, ref - state) < 3e-2
