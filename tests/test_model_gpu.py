"""The CUDA block path (hand-written forward and backward) against the PyTorch oracle on a small model."""
import os

import pytest
import torch

from conftest import rel_err

pytestmark = pytest.mark.gpu


def _small_cfg(after_mod_norm=True, head_dim=64, window=(16, 16)):
    from aeris_gb_b200.models.aeris import AerisConfig
    return AerisConfig(img=(32, 64), window=window, in_channels=20, out_channels=8, dim=128, heads=2,
                       head_dim=head_dim, mlp_dim=256, n_layers=2, sublayers=2, after_mod_norm=after_mod_norm,
                       norm_eps=1e-3, chunk_windows=3)


@pytest.mark.parametrize("after_mod_norm", [True, False])
def test_fused_model_matches_oracle(after_mod_norm):
    from aeris_gb_b200.models.aeris import AerisModel
    torch.manual_seed(1)
    cfg = _small_cfg(after_mod_norm)
    model = AerisModel(cfg).cuda()
    for n, p in model.named_parameters():
        if "modulation" in n and p.dim() == 2:
            torch.nn.init.normal_(p, std=0.05)
    x = torch.randn(2, 32, 64, cfg.in_channels, device="cuda")
    t = torch.tensor([0.3, 1.2], device="cuda")
    params = [p for p in model.parameters() if p.requires_grad]

    def run(force_oracle):
        os.environ["AERIS_FORCE_ORACLE"] = "1" if force_oracle else "0"
        for p in params:
            p.grad = None
        xin = x.clone().requires_grad_(True)
        y = model(xin, t)
        (y * torch.linspace(-1, 1, y.numel(), device="cuda").view_as(y)).sum().backward()
        return y.detach(), xin.grad, [p.grad.clone() if p.grad is not None else None for p in params]

    try:
        y0, gx0, g0 = run(True)
        y1, gx1, g1 = run(False)
    finally:
        os.environ.pop("AERIS_FORCE_ORACLE", None)
    assert rel_err(y1, y0) < 3e-2
    assert rel_err(gx1, gx0) < 5e-2
    names = [n for n, p in model.named_parameters() if p.requires_grad]
    for n, a, b in zip(names, g1, g0):
        if b is None or b.float().norm() == 0:
            continue
        assert a is not None, n
        assert rel_err(a, b) < 8e-2, (n, rel_err(a, b))


def test_fused_model_with_rope_matches_oracle():
    """Optional 2-D rotary embedding: the CUDA path (rotation applied to the qkv chunks, inverse rotation of their
    gradients) against the PyTorch formulation."""
    from aeris_gb_b200.models.aeris import AerisModel
    torch.manual_seed(2)
    cfg = _small_cfg()
    cfg.use_rope = True
    model = AerisModel(cfg).cuda()
    for n, p in model.named_parameters():
        if "modulation" in n and p.dim() == 2:
            torch.nn.init.normal_(p, std=0.05)
    x = torch.randn(2, 32, 64, cfg.in_channels, device="cuda")
    t = torch.tensor([0.3, 1.2], device="cuda")
    params = [p for p in model.parameters() if p.requires_grad]

    def run(force_oracle):
        os.environ["AERIS_FORCE_ORACLE"] = "1" if force_oracle else "0"
        for p in params:
            p.grad = None
        y = model(x, t)
        (y * torch.linspace(-1, 1, y.numel(), device="cuda").view_as(y)).sum().backward()
        return y.detach(), [p.grad.clone() if p.grad is not None else None for p in params]

    try:
        y0, g0 = run(True)
        y1, g1 = run(False)
        cfg.use_rope = False
        y2, _ = run(True)
    finally:
        os.environ.pop("AERIS_FORCE_ORACLE", None)
    assert rel_err(y1, y0) < 3e-2
    assert rel_err(y2, y0) > 1e-3          # the embedding does change the result
    for a, b in zip(g1, g0):
        if b is None or b.float().norm() == 0:
            continue
        assert rel_err(a, b) < 8e-2


def test_wide_block_dim5120_matches_oracle():
    """The block dimensions of the 13 B-class configuration (dim 5120, 40 heads x 128, 30 x 30 windows) on a small
    image: forward and input gradient of the CUDA path against the PyTorch formulation."""
    from aeris_gb_b200.models.aeris import AerisConfig, AerisModel
    torch.manual_seed(4)
    cfg = AerisConfig(img=(60, 120), window=(30, 30), in_channels=20, out_channels=8, dim=5120, heads=40, head_dim=128,
                      mlp_dim=13824, n_layers=2, sublayers=1, norm_eps=1e-3, chunk_windows=3)
    model = AerisModel(cfg).cuda()
    for n, p in model.named_parameters():
        if "modulation" in n and p.dim() == 2:
            torch.nn.init.normal_(p, std=0.02)
    x = torch.randn(1, 60, 120, cfg.in_channels, device="cuda")
    t = torch.tensor([0.7], device="cuda")

    def run(force_oracle):
        os.environ["AERIS_FORCE_ORACLE"] = "1" if force_oracle else "0"
        model.zero_grad(set_to_none=True)
        xin = x.clone().requires_grad_(True)
        y = model(xin, t)
        (y * torch.linspace(-1, 1, y.numel(), device="cuda").view_as(y)).sum().backward()
        return y.detach(), xin.grad, model.layers[0].modulelist[0][3].w2.weight.grad.clone()

    try:
        y0, gx0, gw0 = run(True)
        y1, gx1, gw1 = run(False)
    finally:
        os.environ.pop("AERIS_FORCE_ORACLE", None)
    assert rel_err(y1, y0) < 3e-2
    assert rel_err(gx1, gx0) < 6e-2
    assert rel_err(gw1, gw0) < 8e-2


def test_train_step_raises_on_a_device_timeout_instead_of_stepping():
    """A bounded device wait that runs out (here: a wait on a flag that nothing sets, queued ahead of the step) must
    surface as KernelError from train_step before the optimizer touches the weights; the trainer stays usable."""
    import ctypes
    from aeris_gb_b200.engine.optim import OptimConfig
    from aeris_gb_b200.engine.trainer import DiffusionConfig, Trainer
    from aeris_gb_b200.ops import lib as L
    cfg = _small_cfg()
    tr = Trainer(cfg, OptimConfig(), DiffusionConfig(cond_channels=cfg.in_channels - cfg.out_channels), "cuda:0")
    x = torch.randn(1, 32, 64, cfg.out_channels).pin_memory()
    c = torch.randn(1, 32, 64, cfg.in_channels - cfg.out_channels).pin_memory()
    tr.train_step(x, c)
    before = [p.detach().clone() for p in tr.model.parameters()]
    steps = tr.opt.step_count
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    rc = L.lib().aeris_wait_flag(L.ptr(flag), ctypes.c_uint(1), L.ptr(L.status_word()), ctypes.c_double(0.3),
                                 L.stream_ptr())
    assert rc == 0
    with pytest.raises(L.KernelError, match="peer signal"):
        tr.train_step(x, c)
    assert tr.opt.step_count == steps
    assert all(torch.equal(a, b.detach()) for a, b in zip(before, tr.model.parameters()))
    assert all(float(g.abs().max()) == 0.0 for g in tr.opt.grad_buffers())
    loss = tr.train_step(x, c)              # status cleared, gradients dropped: the next step runs normally
    assert loss == loss and tr.opt.step_count == steps + 1
