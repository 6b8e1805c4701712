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
