"""Real-data path of the inference entry points on a tiny ``[T, 73, H + 1, W]`` store."""
import json
import os
import subprocess
import sys

import numpy as np
import torch

from aeris_gb_b200.data import era5 as E
from aeris_gb_b200.data.inference_data import InferenceData, RolloutWriter, strided_indices
from aeris_gb_b200.diffusion.rollout import Forecaster, SamplerConfig

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
H, W, T = 16, 32, 7


def _make_store(tmp):
    rng = np.random.default_rng(0)
    data = rng.normal(size=(T, 73, H + 1, W)).astype(np.float32) * 3 + 1
    names = E.variable_names(73)
    sst = names.index("sea_surface_temperature")
    data[:, sst, 3:6, 4:9] = np.nan                              # land
    np.save(tmp / "test.npy", data)
    for f, lo, hi in (("normalize_mean", -1, 1), ("normalize_std", 0.5, 2), ("normalize_diff_mean_6", -0.1, 0.1),
                      ("normalize_diff_std_6", 0.5, 1.5)):
        np.savez(tmp / f"{f}.npz", **{n: np.float32(rng.uniform(lo, hi)) for n in names})
    return data, names


def test_strided_initial_conditions_split_over_replicas():
    all_ic, mine = strided_indices(n_times=20, steps=3, dt=1, stride=4, dp_rank=1, dp=2)
    assert all_ic == [0, 4, 8, 12, 16] and mine == [4, 12]


def test_rollout_on_file_data_matches_a_numpy_restatement(tmp_path):
    data, names = _make_store(tmp_path)
    steps, C = 2, 70
    d = InferenceData(str(tmp_path / "test.npy"), str(tmp_path), (H, W), wp=(1, 2), wp_rank=(0, 1), interval=6,
                      rollout_steps=steps, out_channels=C)
    smp = d.sample(1)
    st = d.ds.stats
    wb = W // 2
    # the block: pole row dropped, right half, channels last, SST holes filled (no NaN left)
    raw = d.ds.fill_sst(data[1:1 + steps + 1].copy())
    blk = lambda a: np.moveaxis(a[..., 1:, wb:], -3, -1)
    assert torch.isfinite(smp["state"]).all()
    np.testing.assert_allclose(smp["state"].numpy(), blk(raw[0, :C]), rtol=1e-6)
    np.testing.assert_allclose(smp["truth"].numpy(), blk(raw[1:, :C]), rtol=1e-6)
    r, gp, lsm = names.index("toa_incident_solar_radiation"), names.index("geopotential_at_surface"), names.index("land_sea_mask")
    rad = (raw[:, r:r + 1] - st.x_means[r:r + 1]) / st.x_stds[r:r + 1]
    stat = np.concatenate([(raw[0, i:i + 1] - st.x_means[i:i + 1]) / st.x_stds[i:i + 1] for i in (gp, lsm)], axis=0)
    want_f = np.stack([np.concatenate([rad[k], stat, rad[k + 1]], axis=0) for k in range(steps)])
    np.testing.assert_allclose(smp["forcing"].numpy(), blk(want_f), rtol=1e-5, atol=1e-6)

    # a stand-in network that depends on the noisy state, the condition and the forcing
    def fake(model_in, t):
        return 0.3 * model_in[..., :C] - 0.1 * model_in[..., C:2 * C] + model_in[..., -1:] * 0.05 + t.view(-1, 1, 1, 1)
    sampler = SamplerConfig(n_steps=3, heun=True)
    fc = Forecaster(fake, d.stats("cpu"), sampler, C)
    g = torch.Generator().manual_seed(5)
    noise = [torch.randn(1, H, wb, C, generator=g) for _ in range(steps)]
    x = smp["state"].unsqueeze(0)
    outs = []
    for k in range(steps):
        x = fc.step(x, smp["forcing"][k].unsqueeze(0), x_init=noise[k] * sampler.sigma_data)
        outs.append(x[0].numpy())
    # numpy restatement of the reference loop (pp_generate.py:113-119, 298-333)
    xm, xs = st.x_means[:C].reshape(-1), st.x_stds[:C].reshape(-1)
    tm, ts_ = st.t_means[:C].reshape(-1), st.t_stds[:C].reshape(-1)
    ramp = np.linspace(0, 1, 3)
    sig = (500.0 ** 0.1 + ramp * (0.2 ** 0.1 - 500.0 ** 0.1)) ** 10
    tt = np.concatenate([np.arctan(sig), [0.0]])
    X_un = blk(raw[0, :C]).astype(np.float64)
    for k in range(steps):
        cond = np.concatenate([(X_un - xm) / xs, blk(want_f[k])], axis=-1)
        x_t = noise[k][0].numpy().astype(np.float64)
        net = lambda xx, t: 0.3 * xx - 0.1 * cond[..., :C] + cond[..., -1:] * 0.05 + t
        for i in range(3):
            s_, t_ = tt[i], tt[i + 1]
            F_s = net(x_t, s_)
            x_e = x_t + (t_ - s_) * F_s
            x_t = x_t + (t_ - s_) * 0.5 * (F_s + net(x_e, t_)) if i < 2 else x_e
        X_un = X_un + (x_t * ts_ + tm)
        np.testing.assert_allclose(outs[k], X_un, rtol=2e-4, atol=2e-4)


def test_rollout_writer_layout(tmp_path):
    w = RolloutWriter(str(tmp_path), "r", (1, 0), n_ic=2, steps=1, members=3, C=4, hb=2, wb=5)
    w.put(1, 1, torch.arange(3 * 2 * 5 * 4, dtype=torch.float32).view(3, 2, 5, 4))
    p = w.close()
    a = np.load(p) if p.endswith(".npy") else None
    if a is not None:
        assert a.shape == (2, 2, 3, 4, 2, 5) and a[1, 1, 2, 3, 1, 4] == 3 * 2 * 5 * 4 - 1 and a[0].sum() == 0


def test_wp_inference_cli_reads_the_file_and_writes_the_rollout(tmp_path):
    data, names = _make_store(tmp_path)
    out = tmp_path / "out"
    env = dict(os.environ, AERIS_FORCE_ORACLE="1", PYTHONPATH=ROOT)
    r = subprocess.run([sys.executable, "-m", "aeris_gb_b200.cli.wp_inference", "--experiment", "tiny_cpu", "--members", "2",
                        "--rollout-steps", "2", "--sampler-steps", "2", "--random-init", "--out", str(out),
                        "--data", str(tmp_path / "test.npy"), "--data-root", str(tmp_path), "--stride-ic", "3",
                        "model.img=[16,32]", "model.model_in_channels=144", "model.model_out_channels=70",
                        "model.interval=6"], capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-1500:] + r.stderr[-3000:]
    rec = json.loads(r.stdout.strip().splitlines()[-1])
    assert rec["rollout_steps"] == 2
    # the table of the nine headline variables (first-member RMSE, ensemble-mean RMSE, CRPS, spread/skill per lead time)
    assert "6h" in r.stdout and "12h" in r.stdout and r.stdout.count(" z500:") == 2 and " t2m:" in r.stdout
    files = [f for f in os.listdir(out) if f.startswith("rollout-")]
    assert len(files) == 1
    roll = np.load(out / files[0])
    n_ic = len(range(0, T - 2, 3))
    assert roll.shape == (n_ic, 3, 2, 70, H, W) and np.isfinite(roll).all()
    d = InferenceData(str(tmp_path / "test.npy"), str(tmp_path), (H, W), rollout_steps=2)
    np.testing.assert_allclose(roll[1, 0, 0], d.sample(3)["state"].permute(2, 0, 1).numpy(), rtol=1e-6)
    # the scores the CLI wrote are those of its own rollout against the file's verification fields
    sc = np.load(out / "rollout_err.npy")
    assert sc.shape == (2, 4, 70) and np.isfinite(sc).all()
    truth = torch.stack([d.sample(i)["truth"] for i in range(0, T - 2, 3)]).permute(0, 1, 4, 2, 3).numpy()
    from aeris_gb_b200.diffusion.trigflow import latitude_weights
    w = latitude_weights(H, 0.0).numpy().reshape(1, 1, 1, H, 1)
    mse0 = (w * (roll[:, 1:, 0] - truth) ** 2).mean(axis=(-1, -2)).mean(axis=0)
    np.testing.assert_allclose(sc[:, 0], np.sqrt(mse0), rtol=1e-4)


def test_pp_generate_cli_on_file_data_with_churn_and_dp(tmp_path):
    """Two data-parallel replicas share the strided initial conditions; the churn step and the EMA flag are honoured;
    every replica writes its tile's rollout, whose first frame is the file's state."""
    from aeris_gb_b200.cli.pp_generate import churn_rotation
    s, s_l = churn_rotation(1.2, 4, 2.0, 0.0, float("inf"))
    assert s > 1.2 and s_l > 0 and churn_rotation(1.2, 4, 0.0, 0.0, float("inf")) == (1.2, 0.0)
    _make_store(tmp_path)
    out = tmp_path / "out"
    env = dict(os.environ, AERIS_FORCE_ORACLE="1", PYTHONPATH=ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29747", "-m", "aeris_gb_b200.cli.pp_generate", "--experiment", "tiny_cpu", "--members", "2",
           "--rollout-steps", "1", "--sampler-steps", "2", "--S-churn", "1.0", "--out", str(out),
           "--data", str(tmp_path / "test.npy"), "--data-root", str(tmp_path), "--stride-ic", "3",
           "model.img=[16,32]", "model.model_in_channels=144", "model.model_out_channels=70", "model.interval=6"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-1500:] + r.stderr[-3000:]
    rec = json.loads([l for l in r.stdout.splitlines() if l.startswith("{")][-1])
    assert rec["S_churn"] == 1.0 and rec["initial_conditions"] == 1          # 2 strided ICs over 2 replicas
    files = sorted(f for f in os.listdir(out) if f.startswith("output-"))
    assert len(files) == 2
    d = InferenceData(str(tmp_path / "test.npy"), str(tmp_path), (H, W), rollout_steps=1)
    for dp, f in enumerate(files):
        roll = np.load(out / f)
        assert roll.shape == (1, 2, 2, 70, H, W) and np.isfinite(roll).all()
        np.testing.assert_allclose(roll[0, 0, 1], d.sample(3 * dp)["state"].permute(2, 0, 1).numpy(), rtol=1e-6)
    sc = np.load(out / "pp_rollout_err.npy")
    assert sc.shape == (1, 4, 70) and np.isfinite(sc).all()
