"""Logging helpers, device timers on the host clock, the wandb metric names of the reference, output pre-allocation."""
import numpy as np

from aeris_gb_b200.utils import io as IO
from aeris_gb_b200.utils.timers import DeviceTimers, tflops_per_gpu, wandb_payload


def test_rank_zero_logging_and_printing(capsys, monkeypatch):
    monkeypatch.setenv("RANK", "0")
    IO.log0("hello from rank zero")
    IO.print0("plain", 1)
    monkeypatch.setenv("RANK", "3")
    IO.log0("not shown")
    IO.print0("not shown either")
    IO.print0("rank three speaks", rank=3)
    out = capsys.readouterr().out
    assert "hello from rank zero" in out and "[INFO][aeris.test_utils_cpu]" in out and "plain 1" in out
    assert "not shown" not in out and "rank three speaks" in out


def test_device_timers_fall_back_to_host_time_and_reset():
    t = DeviceTimers(enabled=True, use_nvtx=False)
    with t.region("a"):
        sum(range(1000))
    with t.region("a"):
        pass
    with t.region("b"):
        pass
    r = t.resolve()
    assert set(r) == {"a", "b"} and r["a"] >= 0 and t.resolve() == {}
    off = DeviceTimers(enabled=False)
    with off.region("x"):
        pass
    assert off.resolve() == {}


def test_wandb_metric_names_follow_the_reference():
    d = wandb_payload(7, 140, 55.5, 1.25, loss=0.9, total_norm=2.0, lr=1e-4, stage_norm={3: 0.5}, timers={"fwd": 0.1},
                      pp_rank=2)
    for key in ("train/iter", "train/nimg", "train/tflops_s_tile", "train/dt/iter", "train/loss", "train/total_norm", "lr",
                "train/stage_norm/stage_norm_3", "train/pp_timers/fwd/rank_2"):
        assert key in d, key
    assert d["train/nimg"] == 140 and d["train/tflops_s_tile"] == 55.5
    assert tflops_per_gpu(1e12, 4, 2.0, 2) == 1.0          # 4 samples x 1 TFLOP in 2 s over 2 GPUs


def test_preallocated_numpy_output(tmp_path):
    a = IO.create_empty_numpy(str(tmp_path / "sub" / "out.npy"), (2, 3, 4))
    a[1] = 5.0
    a.flush()
    b = np.load(tmp_path / "sub" / "out.npy")
    assert b.shape == (2, 3, 4) and b[1].min() == 5.0 and b[0].max() == 0.0
