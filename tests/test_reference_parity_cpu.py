"""The model of this package against the reference's own modules (a copy of its sources under ``baseline/_ref``, see
``baseline/install_ref.py``): same weights in, same outputs and gradients out, in every model mode the reference has
(diffusion with both modulate/norm orders and both embedding layouts, random-time-interval, plain pre-norm)."""
import os
import sys
from types import SimpleNamespace

import pytest
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from baseline import harness as HN  # noqa: E402

pytestmark = pytest.mark.skipif(HN.reference_available() is not None, reason="no copy of the reference under baseline/_ref")

H, W, WS, D, C_IN, C_OUT = 16, 32, (8, 8), 32, 10, 4


@pytest.fixture(scope="module")
def one_rank_group():
    from conftest import free_port
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(free_port()))
    dist.init_process_group("gloo", rank=0, world_size=1)
    yield dist.group.WORLD
    dist.destroy_process_group()


CASES = {
    "diffusion_layerwise_modnorm": dict(diffusion=True, rit=False, layerwise=True, after=True, sub=1),
    "diffusion_shared_normmod": dict(diffusion=True, rit=False, layerwise=False, after=False, sub=2),
    "rit": dict(diffusion=False, rit=True, layerwise=False, after=False, sub=1),
    "plain_one_block": dict(diffusion=False, rit=False, layerwise=False, after=False, sub=1),
    "plain_two_blocks": dict(diffusion=False, rit=False, layerwise=False, after=False, sub=2),
}


@pytest.mark.parametrize("name", list(CASES))
def test_same_weights_same_function(name, one_rank_group):
    from aeris_gb_b200.models.aeris import AerisConfig, AerisModel
    c = CASES[name]
    SW, _ = HN._ref_modules()
    torch.manual_seed(0)
    rcfg = SimpleNamespace(model=SimpleNamespace(sinusoidal_emb_max_period=10_000,
                                                 layerwise_t_emb_after_mod_norm=c["after"]))
    kw = dict(rit=c["rit"], diffusion=c["diffusion"], layerwise_t_emb=c["layerwise"])
    f32 = torch.float32
    rin = SW.ParallelSwinInputStage(rcfg, C_IN, D, data_dtype=f32, model_dtype=f32, emb_norm=False, **kw)
    rl = [SW.ParallelSwinLayer(rcfg, D, 2, 16, "pre", 48, WS, 10_000, f32, "flash", sublayers=c["sub"], **kw)
          for _ in range(3)]
    rout = SW.ParallelSwinOutputStage(rcfg, D, C_OUT, "pre", **kw)
    for mod in [rin, *rl, rout]:
        for n, p in mod.named_parameters():
            if p.dim() == 1 and "bias" not in n:
                torch.nn.init.uniform_(p, 0.5, 1.5)          # norm weights away from 1
    cfg = AerisConfig(img=(H, W), window=WS, in_channels=C_IN, out_channels=C_OUT, dim=D, heads=2, head_dim=16, mlp_dim=48,
                      n_layers=3, sublayers=c["sub"], layerwise_t_emb=c["layerwise"], after_mod_norm=c["after"],
                      diffusion=c["diffusion"], rit=c["rit"], model_dtype=f32, ape_row_offset=1)
    ours = AerisModel(cfg)
    sd = {f"input_stage.{k}": v for k, v in rin.state_dict().items()}
    for i, l in enumerate(rl):
        sd.update({f"layers.{i}.{k}": v for k, v in l.state_dict().items()})
    sd.update({f"output_stage.{k}": v for k, v in rout.state_dict().items()})
    missing, unexpected = ours.load_state_dict(sd, strict=False)
    assert not missing and all("rope" in u for u in unexpected), (missing, unexpected)

    g = torch.Generator().manual_seed(1)
    x = torch.randn(1, H, W, C_IN, generator=g)
    wgt = torch.randn(1, H, W, C_OUT, generator=g)
    t = torch.tensor([0.7]) if c["diffusion"] else (torch.tensor([12.0]) if c["rit"] else None)
    # reference: its stages on its own token layout, the odd layers on the shifted partition
    lay = HN.Layout(H, W, WS, "cpu")
    rin.ape_generated = lay.partition(HN._ape_image(SW, C_IN, H, W, "cpu"))
    tok = lay.partition(x[0])
    if c["diffusion"] or c["rit"]:
        h, dt = rin(tok, None, interval=t.view(1, 1))
    else:
        h, dt = rin(tok, None), None
    for i, layer in enumerate(rl):
        if i % 2 == 1:
            h = HN._Permute.apply(h, lay.up, lay.down)
        h = layer(h, None, dt, one_rank_group)
        if i % 2 == 1:
            h = HN._Permute.apply(h, lay.down, lay.up)
    y_ref = rout(h, None, dt, one_rank_group)
    (y_ref * lay.partition(wgt[0])).sum().backward()
    # this package
    y = ours(x, t)
    (y * wgt).sum().backward()
    y_ref_img = torch.empty(H * W, C_OUT)
    y_ref_img[lay.pixel_of] = y_ref.detach().reshape(-1, C_OUT)
    assert torch.allclose(y[0].reshape(-1, C_OUT), y_ref_img, atol=2e-5, rtol=1e-4)
    ref_grads = {f"input_stage.{k}": p.grad for k, p in rin.named_parameters()}
    for i, l in enumerate(rl):
        ref_grads.update({f"layers.{i}.{k}": p.grad for k, p in l.named_parameters()})
    ref_grads.update({f"output_stage.{k}": p.grad for k, p in rout.named_parameters()})
    checked = 0
    for k, p in ours.named_parameters():
        gr = ref_grads.get(k)
        if gr is None or p.grad is None:
            continue
        assert torch.allclose(p.grad, gr, atol=5e-5, rtol=2e-3), (k, (p.grad - gr).abs().max())
        checked += 1
    assert checked >= 10
