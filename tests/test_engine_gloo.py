"""The pipeline engine on CPU ranks (gloo): PP / WP / DP / overlapped schedule / distributed optimizer all have to
reproduce the single-process result; checkpoints written per logical stage reload into any pipeline split."""
import os
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from aeris_gb_b200.engine.optim import OptimConfig
from aeris_gb_b200.engine.pipeline import EngineConfig, ParallelEngine
from aeris_gb_b200.engine.trainer import DiffusionConfig
from aeris_gb_b200.models.aeris import AerisConfig
from aeris_gb_b200.parallel.topology import ProcessGrid

IMG, CH, CC = (16, 32), 6, 4


def _cfg(wp=(1, 1), sp=1, layerwise=True, tp=1):
    """``layerwise``: True / False = diffusion with per-layer / shared noise embedding; "rit" = random-time-interval
    regression (no noise, the condition is the model input)."""
    rit = layerwise == "rit"
    return AerisConfig(img=IMG, window=(8, 8), in_channels=CC if rit else CH + CC, out_channels=CH, dim=32, heads=2,
                       head_dim=16, mlp_dim=64, n_layers=4, sublayers=1, model_dtype=torch.float32, wp=wp, sp=sp,
                       norm_eps=1e-5, layerwise_t_emb=layerwise is True, after_mod_norm=not rit, diffusion=not rit,
                       rit=rit, tp=tp)


def _field(seed, C):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(1, IMG[0], IMG[1], C, generator=g)


def _block(img, eng):
    hb, wb = IMG[0] // eng.grid.WP_Y, IMG[1] // eng.grid.WP_X
    return img[:, eng.c.wp_y * hb:(eng.c.wp_y + 1) * hb, eng.c.wp_x * wb:(eng.c.wp_x + 1) * wb].contiguous()


def _sample_index(eng):
    it, mb = divmod(eng.loads, eng.GAS)
    return (it * eng.GAS + mb) * eng.grid.DP + eng.c.dp


def _data_fn(eng):
    i = _sample_index(eng)
    item = (_block(_field(1000 + i, CC), eng), _block(_field(2000 + i, CH), eng))
    if eng.cfg.rit and not eng.cfg.diffusion:
        item += (torch.tensor([float((6, 12, 24)[i % 3])]),)
    return item


def _noise_fn(eng):
    return _block(_field(3000 + _sample_index(eng), CH), eng)


def _run(rank, world, port, PP, WP, gas, overlap, distopt, iters, out_dir, ckpt_dir, resume, SP=1, layerwise=True,
         TP=1):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    if world > 1:
        dist.init_process_group("gloo", rank=rank, world_size=world)
    grid = ProcessGrid(world, PP=PP, WP_Y=WP[0], WP_X=WP[1], SP=SP)
    ecfg = EngineConfig(gas=gas, overlap_p2p=overlap, dist_optimizer=distopt, checkpoint_dir=ckpt_dir,
                        checkpoint_every=10 ** 9, init_policy=dict(skip=True), seed=5)
    torch.manual_seed(0)
    eng = ParallelEngine(_cfg(WP, SP, layerwise, TP), OptimConfig(lr=0.5, eps=1.0, lr_rampup_img=0, grad_clip_max_norm=0.5, weight_decay=0.0),
                         DiffusionConfig(grad_scale_parity=False, cond_channels=CC), ecfg, grid, rank, "cpu",
                         data_fn=_data_fn, groups={} if world == 1 else None)
    # identical initial weights regardless of the split: every logical stage is seeded by its own index
    from aeris_gb_b200.parallel.tensor import full_state_dict, shard_tensor, tp_kind
    for st, sd in eng.module.logical_state_dicts().items():
        g = torch.Generator().manual_seed(100 + st)
        for k, v in sd.items():
            if v.dtype.is_floating_point and "inv_freq" not in k:
                kind = tp_kind(k) if TP > 1 else None
                if kind is None:
                    v.copy_(torch.randn(v.shape, generator=g) * 0.1)
                else:       # this rank's shard of the full-size draw
                    shape = (v.shape[0] * TP, v.shape[1]) if kind == "w1" else (v.shape[0], v.shape[1] * TP)
                    v.copy_(shard_tensor(kind, torch.randn(shape, generator=g) * 0.1, TP, eng.cfg.tp_rank))
    if TP > 1:
        from aeris_gb_b200.engine.tp_optim import TPOptimizer
        eng.opt = TPOptimizer(eng.module, eng.ocfg, "cpu", eng.groups.get("weight"), eng.groups["tp"],
                              eng.groups.get("tp_ortho"))
    else:
        eng.opt = type(eng.opt)(eng.module, eng.ocfg, *([eng.groups.get("weight"), True] if distopt else []))
    eng.noise_fn = _noise_fn
    eng.t_fn = lambda e: torch.tensor([0.2 + 0.13 * (_sample_index(e) % 9)])
    eng.keep_grads = True
    if resume:
        assert eng.load_checkpoint()
        eng.loads = eng.opt.step_count * gas
    losses = []
    for _ in range(iters):
        eng.exec_schedule()
        losses.append(eng.tot_loss)
    if ckpt_dir and not resume:
        eng.save_checkpoint()
    final_sd, final_grads = eng.module.state_dict(), (eng.last_grads if not distopt else {})
    if TP > 1:          # shards -> full tensors (collective over the tensor-parallel group)
        final_sd = full_state_dict(final_sd, eng.groups["tp"])
        final_grads = full_state_dict(final_grads, eng.groups["tp"])
    if eng.c.dp == 0 and eng.c.wp_y == 0 and eng.c.wp_x == 0 and eng.c.sp == 0:
        torch.save({"sd": {st: {k: v.clone() for k, v in sd.items()}
                           for st, sd in eng.module.logical_state_dicts(final_sd).items()},
                    "grads": eng.module.logical_state_dicts(final_grads) if not distopt else {},
                    "loss": losses, "norm": eng.total_norm}, os.path.join(out_dir, f"pp{eng.c.pp}.pt"))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def _launch(world, **kw):
    out = tempfile.mkdtemp()
    from conftest import free_port
    port = free_port()
    args = (world, port, kw["PP"], kw["WP"], kw["gas"], kw.get("overlap", False), kw.get("distopt", False),
            kw["iters"], out, kw.get("ckpt_dir"), kw.get("resume", False), kw.get("SP", 1), kw.get("layerwise", True),
            kw.get("TP", 1))
    if world == 1:
        _run(0, *args)
    else:
        mp.spawn(_run, args=args, nprocs=world, join=True)
    merged, loss, norm = {}, None, None
    grads = {}
    for f in sorted(os.listdir(out)):
        d = torch.load(os.path.join(out, f), weights_only=True)
        merged.update(d["sd"])
        grads.update(d["grads"])
        if d["loss"] and any(l != 0.0 for l in d["loss"]):
            loss = d["loss"]
        norm = d["norm"]
    _launch.last_grads = grads
    return merged, loss, norm


def _assert_same(a, b, tol=2e-5):
    assert a.keys() == b.keys()
    for st in a:
        for k in a[st]:
            assert torch.allclose(a[st][k], b[st][k], atol=tol, rtol=1e-4), (st, k, (a[st][k] - b[st][k]).abs().max())


@pytest.fixture(scope="module")
def single():
    return _launch(1, PP=1, WP=(1, 1), gas=4, iters=2)


def test_pp2_wp2_with_tensor_parallel_mlp_matches_single_process(single):
    """The MLP weights of every block split over the two window-parallel ranks of each pipeline stage."""
    sd, loss, norm = _launch(4, PP=2, WP=(1, 2), gas=4, iters=2, TP=2)
    _assert_same(sd, single[0], tol=5e-5)
    assert loss == pytest.approx(single[1], rel=1e-4)
    assert norm == pytest.approx(single[2], rel=1e-4)


def test_sp2_with_tensor_parallel_mlp_over_the_sequence_pair_matches_single_process(single):
    """SP 2 with the MLP weights split over the sequence-parallel pair (the tensor-parallel group is the SP group)."""
    sd, loss, norm = _launch(2, PP=1, WP=(1, 1), SP=2, gas=4, iters=2, TP=2)
    _assert_same(sd, single[0], tol=5e-5)
    assert loss == pytest.approx(single[1], rel=1e-4)
    assert norm == pytest.approx(single[2], rel=1e-4)


def test_pp3_matches_single_process(single):
    sd, loss, norm = _launch(3, PP=3, WP=(1, 1), gas=4, iters=2)
    _assert_same(sd, single[0])
    assert loss == pytest.approx(single[1], rel=1e-4)
    assert norm == pytest.approx(single[2], rel=1e-4)


def test_pp3_shared_noise_embedding_gets_its_gradient_from_every_stage():
    """One embedding network on the first stage (layerwise_t_emb off): its output dt feeds every stage, so its
    gradient has to travel back up the pipeline with that of the activations (parallel_engine.py:1052-1068)."""
    ref = _launch(1, PP=1, WP=(1, 1), gas=4, iters=2, layerwise=False)
    ref_grads = _launch.last_grads
    sd, loss, norm = _launch(3, PP=3, WP=(1, 1), gas=4, iters=2, overlap=True, layerwise=False)
    g = _launch.last_grads
    k = "latent_embed.w1.weight"
    assert ref_grads[0][k].abs().max() > 0
    assert torch.allclose(g[0][k], ref_grads[0][k], atol=1e-6, rtol=1e-4)
    _assert_same(sd, ref[0])
    assert norm == pytest.approx(ref[2], rel=1e-4)


def test_pp2_wp2_random_time_interval_mode_matches_single_process():
    """Deterministic regression conditioned on the embedded forecast interval (rit): the interval embedding on the
    first stage is trained through every stage of the pipeline."""
    ref = _launch(1, PP=1, WP=(1, 1), gas=3, iters=2, layerwise="rit")
    ref_grads = _launch.last_grads
    sd, loss, norm = _launch(4, PP=2, WP=(1, 2), gas=3, iters=2, overlap=True, layerwise="rit")
    assert ref_grads[0]["interval_embed.weight"].abs().max() > 0
    assert torch.allclose(_launch.last_grads[0]["interval_embed.weight"], ref_grads[0]["interval_embed.weight"],
                          atol=1e-6, rtol=1e-4)
    _assert_same(sd, ref[0])
    assert loss == pytest.approx(ref[1], rel=1e-4)


def test_pp2_overlapped_wp2_matches_single_process(single):
    sd, loss, _ = _launch(4, PP=2, WP=(1, 2), gas=4, iters=2, overlap=True)
    _assert_same(sd, single[0])
    assert loss == pytest.approx(single[1], rel=1e-4)


def test_ulysses_sp2_with_wp2_matches_single_process(single):
    sd, loss, _ = _launch(4, PP=1, WP=(1, 2), SP=2, gas=4, iters=2)
    _assert_same(sd, single[0])
    assert loss == pytest.approx(single[1], rel=1e-4)


def test_dp2_distributed_optimizer_matches_single_process(single):
    sd, _, _ = _launch(2, PP=1, WP=(1, 1), gas=2, iters=2, distopt=True)
    _assert_same(sd, single[0])


def test_checkpoint_roundtrip_across_pipeline_splits(single):
    ck = tempfile.mkdtemp()
    _launch(1, PP=1, WP=(1, 1), gas=4, iters=1, ckpt_dir=ck)
    assert sorted(os.listdir(ck)) == [f"checkpoint_PP{i}.pth" for i in range(6)]
    d = torch.load(os.path.join(ck, "checkpoint_PP1.pth"), weights_only=True)
    assert set(d) == {"cur_nimg", "model_state_dict", "main_model_state_dict", "optimizer_state_dict", "ema_state_dict",
                      "integrity"}     # the five reference keys plus the payload check
    assert "modulelist.0.1.to_qkv.weight" in d["model_state_dict"] and d["cur_nimg"] == 4
    # resume the second iteration on a 2-stage pipeline: must land on the single-process 2-iteration weights
    sd, _, _ = _launch(2, PP=2, WP=(1, 1), gas=4, iters=1, ckpt_dir=ck, resume=True)
    _assert_same(sd, single[0])


def test_dp2_distributed_optimizer_checkpoint_resumes(single):
    """The sharded optimizer state is gathered into the per-stage files and scattered back: one iteration, save,
    reload on two ranks, second iteration lands on the single-process two-iteration weights."""
    ck = tempfile.mkdtemp()
    _launch(2, PP=1, WP=(1, 1), gas=2, iters=1, distopt=True, ckpt_dir=ck)
    assert sorted(os.listdir(ck)) == [f"checkpoint_PP{i}.pth" for i in range(6)]
    sd, _, _ = _launch(2, PP=1, WP=(1, 1), gas=2, iters=1, distopt=True, ckpt_dir=ck, resume=True)
    _assert_same(sd, single[0])


def test_checkpoint_with_the_references_optimizer_layout_loads(tmp_path):
    """A file whose ``optimizer_state_dict`` is what ``torch.optim.AdamW.state_dict()`` returns for the stage's
    parameter list (no names, positions only: parallel_engine.py:1128-1137) resumes; a foreign layout is refused
    without touching the model."""
    from aeris_gb_b200.engine.checkpoint import load_stage_checkpoint, save_stage_checkpoint
    from aeris_gb_b200.engine.optim import FlatOptimizer
    from aeris_gb_b200.models.aeris import AerisModel
    torch.manual_seed(0)
    model = AerisModel(_cfg())
    opt = FlatOptimizer(model, OptimConfig())
    for s in opt.segments:
        s.m.normal_(); s.v.uniform_()
    opt.step_count, opt.cur_nimg = 7, 28
    save_stage_checkpoint(str(tmp_path), model, opt)
    m_ref = {k: v.clone() for k, v in opt.state_dict()["exp_avg"].items()}
    # rewrite stage 1 the way torch would: state keyed by position, parameters without names
    f = os.path.join(tmp_path, "checkpoint_PP1.pth")
    ck = torch.load(f, weights_only=True)
    layer = torch.nn.ModuleList([p for p in [model.layers[0]]])[0]
    plist = [torch.nn.Parameter(p.detach().float().clone()) for _, p in layer.named_parameters()]
    ref_opt = torch.optim.AdamW(plist, lr=1e-3)
    for p in plist:
        p.grad = torch.zeros_like(p)
    ref_opt.step()
    tsd = ref_opt.state_dict()
    own = ck["optimizer_state_dict"]
    for i, name in enumerate(own["param_names"]):
        if i in own["state"]:
            tsd["state"][i]["exp_avg"] = own["state"][i]["exp_avg"]
            tsd["state"][i]["exp_avg_sq"] = own["state"][i]["exp_avg_sq"]
            tsd["state"][i]["step"] = torch.tensor(7.0)
        else:
            tsd["state"].pop(i, None)
    assert "param_names" not in tsd
    ck["optimizer_state_dict"] = tsd
    ck.pop("integrity")
    torch.save(ck, f)
    model2 = AerisModel(_cfg())
    opt2 = FlatOptimizer(model2, OptimConfig())
    assert load_stage_checkpoint(str(tmp_path), model2, opt2, "cpu")
    assert opt2.step_count == 7 and opt2.cur_nimg == 28
    got = opt2.state_dict()["exp_avg"]
    for k in m_ref:
        assert torch.equal(got[k], m_ref[k]), k
    # an optimizer section in some other layout: refused, nothing loaded
    ck["optimizer_state_dict"] = {"step": 7, "moments": {}}
    torch.save(ck, f)
    model3 = AerisModel(_cfg())
    before = {k: v.clone() for k, v in model3.state_dict().items()}
    assert not load_stage_checkpoint(str(tmp_path), model3, FlatOptimizer(model3, OptimConfig()), "cpu")
    assert all(torch.equal(v, before[k]) for k, v in model3.state_dict().items())


def test_inference_engine_releases_the_training_state_of_its_bf16_parameters():
    """Forward-only engine: fp32 masters, gradient buffers, Adam moments and EMA of the bf16 blocks are freed after
    construction, the parameters keep their values, and a network evaluation still runs."""
    from aeris_gb_b200.engine.inference import InferenceEngine
    cfg = _cfg()
    cfg.model_dtype = torch.bfloat16
    grid = ProcessGrid(1, PP=1)
    torch.manual_seed(0)
    eng = InferenceEngine(cfg, OptimConfig(use_ema=False), DiffusionConfig(cond_channels=CC),
                          EngineConfig(gas=1, init_policy=dict(skip=True)), grid, 0, "cpu", members=2, groups={})
    lp = [s for s in eng.opt.segments if s.low_precision]
    assert lp and all(s.master is None and s.grad is None and s.m is None and s.v is None for s in lp)
    blocks = [p for n, p in eng.module.named_parameters() if "to_qkv" in n]
    assert blocks and all(p.dtype == torch.bfloat16 and not hasattr(p, "main_grad") and p.abs().sum() > 0 for p in blocks)
    rows = eng.tokens
    g = torch.Generator().manual_seed(1)
    out = eng.exec_schedule([torch.randn(rows, CH + CC, generator=g) for _ in range(2)], torch.tensor([0.7]))
    assert len(out) == 2 and out[0].shape == (rows, CH) and torch.isfinite(out[0]).all()
    assert not torch.equal(out[0], out[1])
