import os
import tempfile

import numpy as np
import pytest
import torch

from aeris_gb_b200.data import era5 as E
from aeris_gb_b200.data.prep import merge as M
from aeris_gb_b200.data.prep import wp_create as WPC
from aeris_gb_b200.data.samplers import AttributeSubset, InfiniteSampler
from aeris_gb_b200.data.store import save_array
from aeris_gb_b200.data.synthetic import SyntheticERA5
from aeris_gb_b200.eval.metrics import EnsembleMetrics, step_sums
from aeris_gb_b200.utils.io import compress_variables


def test_variable_sets():
    assert len(E.variable_names(69)) == 69 and len(E.variable_names(72)) == 72 and len(E.variable_names(73)) == 73
    v = E.variable_names(73)
    assert v[0] == "2m_temperature" and v[69] == "sea_surface_temperature" and v[70] == "toa_incident_solar_radiation"
    g = compress_variables(v)
    assert g["geopotential"][1] == E.LEVELS and g["2m_temperature"] == ([0], [])


def test_crps_pair_sum_matches_bruteforce():
    torch.manual_seed(0)
    m = torch.randn(5, 3, 6, 8, dtype=torch.float64)
    y = torch.randn(3, 6, 8, dtype=torch.float64)
    w = torch.rand(6, dtype=torch.float64)
    s = step_sums(m, y, w)
    brute = (w.view(1, 1, 1, -1, 1) * (m.unsqueeze(1) - m.unsqueeze(0)).abs()).sum(dim=(-2, -1)).sum(dim=(0, 1)) / (2 * 5 * 4)
    assert torch.allclose(s[3], brute)
    assert torch.allclose(s[0], (w.view(1, -1, 1) * (y - m[0]) ** 2).sum(dim=(-1, -2)))


def test_metrics_perfect_ensemble_and_finalize():
    C, H, W = 2, 4, 8
    y = torch.randn(C, H, W)
    em = EnsembleMetrics(rollout_steps=2, n_channels=C, n_pixels=H * W, device="cpu")
    members = y.unsqueeze(0).repeat(3, 1, 1, 1) + 0.1 * torch.randn(3, C, H, W)
    em.update(0, members, y, torch.ones(H))
    em.update(1, members, y, torch.ones(H))
    em.end_initial_condition()
    agg, sc = em.finalize()
    assert agg.shape == (2, 5, C) and sc.shape == (2, 4, C)
    assert (sc[:, 0] < 0.3).all() and (sc[:, 2] >= -1e-9).all()      # small RMSE, non-negative CRPS


def test_dataset_pipeline_with_npy_store():
    d = tempfile.mkdtemp()
    rng = np.random.default_rng(0)
    n, C = 6, 69
    os.makedirs(os.path.join(d, "steps"))
    for i in range(n):
        np.save(os.path.join(d, "steps", f"t{i:03d}.npy"), rng.normal(size=(C, 721, 8)).astype(np.float32))
    merged = M.merge(os.path.join(d, "steps"), os.path.join(d, "merged"), C, shape_hw=(721, 8))
    arr = np.load(merged, mmap_mode="r")
    assert arr.shape == (n, C, 721, 8)
    # statistics files
    names = E.variable_names(C)
    for f, val in (("normalize_mean.npz", 0.5), ("normalize_std.npz", 2.0), ("normalize_diff_mean_6.npz", 0.0),
                   ("normalize_diff_std_6.npz", 4.0)):
        np.savez(os.path.join(d, f), **{v: np.float32(val) for v in names})
    ds = E.ERA5NRMDataset(d, merged, interval=6, channels=C, samples=n - 1)
    ds.open_file()
    x, t = ds[2]
    assert torch.allclose(x, torch.from_numpy((arr[2] - 0.5) / 2.0)) and torch.allclose(t, torch.from_numpy((arr[3] - arr[2]) / 4.0))
    sub = AttributeSubset(ds, [0, 1, 2])
    assert sub.n_channels == C and len(sub) == 3


def test_wp_create_layouts_partition_the_field():
    d = tempfile.mkdtemp()
    a = np.arange(2 * 3 * 721 * 24, dtype=np.float32).reshape(2, 3, 721, 24) + 1
    src = save_array(os.path.join(d, "m"), a, prefer_h5=False)
    for layout in ("strided", "block"):
        files = WPC.create(src, os.path.join(d, layout), 2, 2, window=(8, 4), layout=layout) \
            if 720 % (8 * 2) == 0 else []
        seen = np.concatenate([np.load(f).ravel() for f in files])
        assert sorted(seen.tolist()) == sorted(a[:, :, 1:].ravel().tolist())
    t = WPC.tile_for_rank(a[0], 1, 0, 2, 2, 8, 4, "strided")
    assert t.shape == (3, 360, 12) and t[0, 0, 0] == a[0, 0, 1 + 8, 0]


def test_infinite_sampler_is_rank_strided_and_endless():
    ds = list(range(10))
    s0 = iter(InfiniteSampler(ds, rank=0, num_replicas=2, shuffle=False))
    s1 = iter(InfiniteSampler(ds, rank=1, num_replicas=2, shuffle=False))
    a = [next(s0) for _ in range(12)]
    b = [next(s1) for _ in range(12)]
    assert a[:5] == [0, 2, 4, 6, 8] and b[:5] == [1, 3, 5, 7, 9] and a[5] == 0
    sh = iter(InfiniteSampler(ds, shuffle=True, seed=3))
    drawn = [next(sh) for _ in range(200)]
    assert set(drawn) == set(range(10))          # windowed re-shuffling keeps every element in circulation
    # the order for a seed is that of numpy's default generator (src/aeris/data/samplers.py:35-45): first the shuffled
    # permutation, one windowed swap after every index
    rnd = np.random.default_rng(3)
    order = np.arange(10)
    rnd.shuffle(order)
    expect = []
    for idx in range(25):
        i = idx % 10
        expect.append(int(order[i]))
        j = (i - rnd.integers(5)) % 10
        order[i], order[j] = order[j], order[i]
    assert drawn[:25] == expect


def test_synthetic_dataset_blocks():
    ds = SyntheticERA5(img=(16, 32), cond_channels=3, target_channels=2, wp=(2, 2), wp_rank=(1, 0))
    c, t = ds[0]
    assert c.shape == (8, 16, 3) and t.shape == (8, 16, 2)
    assert torch.equal(ds[4][0], c)      # pool of 4 distinct samples


def test_rollout_to_zarr_v2_store_round_trip(tmp_path):
    """The rollout -> Zarr conversion with the built-in Zarr v2 writer: multi-level variables become
    [time, level, lat, lon] arrays, surface variables [time, lat, lon]; two workers split the files; a write that
    fails transiently is retried."""
    import json
    from aeris_gb_b200.data.era5 import variable_names
    from aeris_gb_b200.data.prep import h52zarr as Z
    variables = variable_names(73)[:70]
    rng = np.random.default_rng(0)
    src = tmp_path / "rollout"
    src.mkdir()
    files, arrays = [], []
    for m in range(3):
        a = rng.standard_normal((4, 70, 6, 8)).astype(np.float32)
        np.save(src / f"member{m}.npy", a)
        files.append(str(src / f"member{m}.npy"))
        arrays.append(a)
    dst = str(tmp_path / "out.zarr")
    for rank in range(2):
        Z.convert(files, dst, variables, rank=rank, world=2, use_zarr_package=False)
    assert json.load(open(os.path.join(dst, ".zgroup"))) == {"zarr_format": 2}
    from aeris_gb_b200.utils.io import compress_variables
    groups = compress_variables(variables)
    name, (idx, levels) = next((k, v) for k, v in groups.items() if v[1])
    for m in range(3):
        got = Z.read_zarr_v2_array(os.path.join(dst, f"member_{m}", name))
        assert got.shape == (4, len(levels), 6, 8) and np.array_equal(got, arrays[m][:, idx])
        meta = json.load(open(os.path.join(dst, f"member_{m}", name, ".zattrs")))
        assert meta["_ARRAY_DIMENSIONS"] == ["time", "level", "latitude", "longitude"]
        surf = Z.read_zarr_v2_array(os.path.join(dst, f"member_{m}", "2m_temperature"))
        assert np.array_equal(surf, arrays[m][:, groups["2m_temperature"][0][0]])
    # retries: two transient failures, then success; a persistent failure is raised after the last attempt
    calls = {"n": 0}

    def flaky():
        calls["n"] += 1
        if calls["n"] < 3:
            raise OSError("stale file handle")
        return "ok"
    assert Z._write_with_retries(flaky, 10, sleep=lambda s: None) == "ok" and calls["n"] == 3
    with pytest.raises(OSError):
        Z._write_with_retries(lambda: (_ for _ in ()).throw(OSError("gone")), 3, sleep=lambda s: None)
