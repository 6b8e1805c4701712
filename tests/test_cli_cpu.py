"""Entry points run end to end on CPU with the tiny configuration."""
import json
import os
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ENV = dict(os.environ, AERIS_FORCE_ORACLE="1", PYTHONPATH=ROOT)


def _run(args, nproc=1, port=29741):
    if nproc == 1:
        cmd = [sys.executable, "-m"] + args
    else:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
               "--master-addr", "127.0.0.1", "--master-port", str(port), "-m"] + args
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=ENV, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-1500:] + r.stderr[-3000:]
    return r.stdout


def test_train_cli_loss_goes_down_and_writes_run_config(tmp_path):
    out = _run(["aeris_gb_b200.cli.train", "experiment=tiny_cpu", "trainer.benchmark_steps=6",
                f"model.checkpoint_dir={tmp_path}", "optimizer.lr=0.003", "trainer.lr_rampup_kimg=0"])
    losses = [float(l.split("loss ")[1].split()[0]) for l in out.splitlines() if " loss " in l]
    assert len(losses) == 6 and losses[-1] < losses[0]
    assert (tmp_path / ".hydra" / "config.yaml").exists()


def test_train_cli_writes_a_profiler_trace(tmp_path):
    out = _run(["aeris_gb_b200.cli.train", "experiment=tiny_cpu", "trainer.benchmark_steps=3", "trainer.profile_steps=[1,2]",
                f"model.checkpoint_dir={tmp_path}"])
    assert "profiler trace written" in out
    trace = tmp_path / "traces" / "trace_rank0_it1-2.json"
    assert trace.exists() and "traceEvents" in trace.read_text()[:2000]


def test_wp_inference_cli(tmp_path):
    out = _run(["aeris_gb_b200.cli.wp_inference", "--experiment", "tiny_cpu", "--members", "3", "--rollout-steps", "2",
                "--sampler-steps", "2", "--random-init", "--out", str(tmp_path)])
    rec = json.loads(out.strip().splitlines()[-1])
    assert rec["model_evals_per_step"] == 3 and rec["rollout_steps"] == 2
    sc = np.load(tmp_path / "rollout_err.npy")
    assert sc.shape == (2, 4, 16) and np.isfinite(sc).all()


def test_pp_generate_cli_two_stage_pipeline():
    out = _run(["aeris_gb_b200.cli.pp_generate", "--experiment", "tiny_cpu", "--PP", "2", "--members", "3",
                "--rollout-steps", "1", "--sampler-steps", "2"], nproc=2)
    rec = json.loads([l for l in out.splitlines() if l.startswith("{")][-1])
    assert rec["PP"] == 2 and rec["network_evaluations"] == 3


def test_resumed_trainer_does_not_replay_the_first_noise_draws(tmp_path):
    """step, save, reload into a fresh trainer, resume: the next noise level and noise differ from those of step 0,
    the step counter that seeds the fused input kernels continues (parallel_engine.py:1155-1156, train.py:247)."""
    import torch
    from aeris_gb_b200.engine.checkpoint import load_stage_checkpoint, save_stage_checkpoint
    from aeris_gb_b200.engine.optim import OptimConfig
    from aeris_gb_b200.engine.trainer import DiffusionConfig, Trainer
    from aeris_gb_b200.models.aeris import AerisConfig
    from aeris_gb_b200.diffusion import trigflow as TF
    cfg = AerisConfig(img=(16, 32), window=(8, 8), in_channels=10, out_channels=4, dim=32, heads=2, head_dim=16,
                      mlp_dim=64, n_layers=2, sublayers=1, model_dtype=torch.float32)
    dc = DiffusionConfig(cond_channels=6)

    def draws(tr):
        t = TF.sample_noise_level(1, dc.sigma_min, dc.sigma_max, dc.sigma_data, generator=tr.nl_rng, device="cpu")
        return t, torch.randn(8, generator=tr.rng)
    fresh = Trainer(cfg, OptimConfig(), dc, "cpu", seed=3)
    t0, z0 = draws(fresh)
    tr = Trainer(cfg, OptimConfig(), dc, "cpu", seed=3)
    g = torch.Generator().manual_seed(0)
    x, c = torch.randn(2, 16, 32, 4, generator=g), torch.randn(2, 16, 32, 6, generator=g)
    tr.train_step(x, c)
    save_stage_checkpoint(str(tmp_path), tr.model, tr.opt)
    tr2 = Trainer(cfg, OptimConfig(), dc, "cpu", seed=3)
    assert load_stage_checkpoint(str(tmp_path), tr2.model, tr2.opt, "cpu")
    tr2.resume(tr2.opt.cur_nimg, gas=2)
    assert tr2.step_count == 1 and tr2.opt.cur_nimg == 2
    t1, z1 = draws(tr2)
    assert not torch.equal(t1, t0) and not torch.equal(z1, z0)


def test_stage_metric_names_follow_the_reference():
    import torch
    from aeris_gb_b200.cli.train import stage_metrics
    from aeris_gb_b200.models.aeris import AerisConfig, SwinLayer
    cfg = AerisConfig(img=(16, 32), window=(8, 8), in_channels=10, out_channels=4, dim=32, heads=2, head_dim=16,
                      mlp_dim=64, n_layers=2, sublayers=1, model_dtype=torch.float32)
    m = stage_metrics({1: SwinLayer(cfg)}, 2.5, 1, 4, {"ForwardPass": 0.1})
    assert set(m) == {"train/stage_norm/stage_norm_1", "train/weight_norm/stage_1/0_modulation_0",
                      "train/weight_norm/stage_1/0_modulation_2", "train/pp_timers/ForwardPass/rank_1"}


def test_reference_benchmark_experiment_trains_at_toy_size():
    """``experiment=benchmark`` (the reference's own benchmark config: random-time-interval regression, overlapped
    pipeline p2p, distributed optimizer) composes and trains with its sizes overridden, PP 2 x WP 2 on four ranks."""
    out = _run(["aeris_gb_b200.cli.train", "experiment=benchmark", "data.synthetic=true", "data.gas=3",
                "trainer.benchmark_steps=3", "model.PP=2", "model.SP=1", "model.WP_X=2", "model.WP_Y=1", "model.dim=32",
                "model.heads=2", "model.head_dim=16", "model.mlp_dim=64", "model.PP_stages=4", "model.window_size=[8,8]",
                "model.img=[16,32]", "model.checkpoint_dir=null", "model.dtype=float32", "model.channels=6",
                "optimizer.lr=0.01", "trainer.lr_rampup_kimg=0"], nproc=4, port=29763)
    losses = [float(l.split("loss ")[1].split()[0]) for l in out.splitlines() if " loss " in l]
    # the synthetic targets are independent standard-normal fields, so the regression loss stays near their variance;
    # what is checked is that the configuration composes, runs its three optimizer steps and reports finite losses
    assert len(losses) == 3 and all(0.5 < l < 1.5 for l in losses)


def test_train_cli_with_tensor_parallel_mlp(tmp_path):
    """``model.TP``: the MLP weights split over the two window-parallel ranks; the run trains, checkpoints (full
    tensors on disk) and a second run resumes from the checkpoint."""
    import torch
    args = ["aeris_gb_b200.cli.train", "experiment=tiny_cpu", "model.WP_X=2", "model.TP=2", "optimizer.lr=0.003",
            "trainer.lr_rampup_kimg=0", f"model.checkpoint_dir={tmp_path}", "trainer.checkpoint_every=2"]
    out = _run(args + ["trainer.benchmark_steps=4"], nproc=2, port=29771)
    losses = [float(l.split("loss ")[1].split()[0]) for l in out.splitlines() if " loss " in l]
    assert len(losses) == 4 and losses[-1] < losses[0]
    ck = torch.load(tmp_path / "checkpoint_PP1.pth", map_location="cpu", weights_only=True)
    w1 = [v for k, v in ck["model_state_dict"].items() if k.endswith("w1.weight")][0]
    assert tuple(w1.shape) == (512, 128)                      # 2 x mlp_dim rows: the gathered, unsharded weight
    out = _run(args + ["trainer.benchmark_steps=6", "model.load=true"], nproc=2, port=29772)
    assert "loaded a checkpoint" in out
    assert len([l for l in out.splitlines() if " loss " in l]) == 2
    # the inference entry point holds whole MLP weights and takes the same files
    out = _run(["aeris_gb_b200.cli.wp_inference", "--experiment", "tiny_cpu", "--checkpoint", str(tmp_path), "--members",
                "2", "--rollout-steps", "1", "--sampler-steps", "2", "model.TP=2"])
    rec = json.loads(out.strip().splitlines()[-1])
    assert rec["rollout_steps"] == 1
    # a numbered copy is addressed by the text in front of its file names (--extra-name)
    for f in list(os.listdir(tmp_path)):
        if f.startswith("checkpoint_PP"):
            os.rename(tmp_path / f, tmp_path / ("it_7_" + f))
    out = _run(["aeris_gb_b200.cli.wp_inference", "--experiment", "tiny_cpu", "--checkpoint", str(tmp_path), "--members",
                "1", "--steps", "1", "--diffusion-steps", "2", "--extra-name", "it_7_"])
    assert json.loads(out.strip().splitlines()[-1])["rollout_steps"] == 1


def test_tensor_parallel_with_data_parallel_replicas_matches_replicated_weights():
    """Four ranks = DP 2 x WP 2 with ``model.TP=2``: every shard is held by two ranks (one per replica), so its
    gradient is reduced over those two only while the replicated parameters are reduced over all four, with one clipping
    norm. The loss curve has to equal the run with replicated MLP weights."""
    args = ["aeris_gb_b200.cli.train", "experiment=tiny_cpu", "model.WP_X=2", "optimizer.lr=0.003",
            "trainer.lr_rampup_kimg=0", "model.checkpoint_dir=null", "trainer.benchmark_steps=3", "model.grad_clip=true",
            "model.grad_clip_max_norm=0.05"]
    curves = []
    for extra, port in ((["model.TP=2"], 29781), ([], 29782)):
        out = _run(args + extra, nproc=4, port=port)
        curves.append([float(l.split("loss ")[1].split()[0]) for l in out.splitlines() if " loss " in l])
    assert len(curves[0]) == 3 and np.allclose(curves[0], curves[1], rtol=2e-4), curves


def test_train_cli_window_sequence_and_tensor_parallel_on_cpu_ranks():
    """``experiment=b200_1p3b_wp4_sp2`` at toy size on four gloo ranks (WP 2 x SP 2, MLP weights split over each SP
    pair): on CPU ranks sequence parallelism runs through the pipeline engine with one stage."""
    out = _run(["aeris_gb_b200.cli.train", "experiment=b200_1p3b_wp4_sp2", "model.TP=2", "model.WP_X=2", "model.WP_Y=1",
                "data.synthetic=true", "data.gas=2", "trainer.benchmark_steps=2", "model.dim=32", "model.heads=2",
                "model.head_dim=16", "model.mlp_dim=64", "model.PP_stages=4", "model.window_size=[8,8]",
                "model.img=[16,32]", "model.checkpoint_dir=null", "model.dtype=float32", "model.channels=6"],
               nproc=4, port=29792)
    losses = [float(l.split("loss ")[1].split()[0]) for l in out.splitlines() if " loss " in l]
    assert len(losses) == 2 and all(0.5 < l < 2.0 for l in losses)


def test_inference_clis_take_the_references_option_spellings():
    """`--steps`, `--diffusion-steps`, `--stride`, `--use-ema`, `--S_churn` ... are accepted as the reference spells them
    (pp_generate.py:28-53, aeris_wp_inference/inference.py:24-41), next to this package's own spellings."""
    out = _run(["aeris_gb_b200.cli.wp_inference", "--experiment", "tiny_cpu", "--members", "2", "--steps", "1",
                "--diffusion-steps", "2", "--stride", "5", "--S_churn", "0.5", "--S_min", "0", "--S_max", "100",
                "--S_noise", "1.003", "--sigma_max", "80", "--sigma_min", "0.3", "--sequence-parallel", "1",
                "--random-init"])
    rec = json.loads(out.strip().splitlines()[-1])
    assert rec["rollout_steps"] == 1 and rec["sampler_steps"] == 2
    out = _run(["aeris_gb_b200.cli.pp_generate", "--experiment", "tiny_cpu", "--PP", "1", "--members", "2", "--steps", "1",
                "--diffusion-steps", "2", "--S_churn", "0.5", "--S_noise", "1.003", "--sigma_max", "80", "--use-ema",
                "--clamp-sst", "--start-sample", "0", "--end-sample", "3"])
    rec = json.loads([l for l in out.splitlines() if l.startswith("{")][-1])
    assert rec["rollout_steps"] == 1 and rec["ema"] is True and rec["S_churn"] == 0.5
