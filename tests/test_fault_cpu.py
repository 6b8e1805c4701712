"""Failure detection without touching a GPU: failures are made on the host (a rank that raises or goes silent, a
corrupted checkpoint, a NaN in a host tensor) and ranks are gloo processes."""
import os
import tempfile
import time

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from aeris_gb_b200.utils.fault import (FaultInjector, Heartbeat, NonFiniteError, RankFailure, StepWatchdog,
                                       check_finite)


def _worker(rank, world, port, out):
    store = dist.TCPStore("127.0.0.1", port, world, is_master=(rank == 0), timeout=__import__("datetime").timedelta(seconds=30))
    hb = Heartbeat(store, rank, world, timeout_s=2.5)
    inj = FaultInjector("silent:rank=1:step=2")
    detected = None
    store.add("ready", 1)                      # start together even when the machine is busy spawning the ranks
    while int(store.add("ready", 0)) < world:
        time.sleep(0.05)
    for step in range(40):
        if not inj.silences(rank, step):
            hb.beat()                          # ranks that have noticed the failure keep beating until all have
        time.sleep(0.3)
        if detected is None:
            try:
                hb.check()
            except RankFailure as e:
                detected = (step, str(e))
                store.add("detected", 1)
        if int(store.add("detected", 0)) >= world - 1:
            break
    with open(os.path.join(out, f"r{rank}.txt"), "w") as f:
        f.write(repr(detected))
    store.add("done", 1)                       # rank 0 owns the store: keep it alive until the others are done
    t0 = time.time()
    while rank == 0 and int(store.add("done", 0)) < world and time.time() - t0 < 30:
        time.sleep(0.1)


def test_heartbeat_detects_a_silent_rank_between_steps():
    out = tempfile.mkdtemp()
    from conftest import free_port
    mp.spawn(_worker, args=(3, free_port(), out), nprocs=3, join=True)
    r0 = open(os.path.join(out, "r0.txt")).read()
    r2 = open(os.path.join(out, "r2.txt")).read()
    assert "ranks [1]" in r0 and "ranks [1]" in r2
    assert open(os.path.join(out, "r1.txt")).read() == "None"   # the silent rank itself sees healthy peers


def test_heartbeat_leaving_rank_is_reported_immediately():
    class Store(dict):
        def set(self, k, v): self[k] = v.encode()
        def get(self, k): return self[k]
        def check(self, ks): return all(k in self for k in ks)
    s = Store()
    a, b = Heartbeat(s, 0, 2, timeout_s=100), Heartbeat(s, 1, 2, timeout_s=100)
    a.beat(); b.beat()
    assert a.dead_ranks() == []
    b.mark_leaving()
    with pytest.raises(RankFailure):
        a.check()


def test_watchdog_and_finite_guard():
    w = StepWatchdog(factor=2.0, warmup=3)
    assert not any(w.observe(1.0) for _ in range(5))
    assert w.observe(5.0)
    check_finite("loss", 1.0)
    with pytest.raises(NonFiniteError):
        check_finite("loss", float("nan"))
    inj = FaultInjector("nan:rank=0:step=2")
    t = inj.poison(torch.ones(4), 0, 2)
    assert torch.isnan(t[0]) and not torch.isnan(inj.poison(torch.ones(4), 0, 1)).any()
    with pytest.raises(RuntimeError):
        FaultInjector("raise:rank=3:step=1").maybe_raise(3, 1)


def test_corrupted_checkpoint_is_rejected_not_half_loaded():
    from aeris_gb_b200.engine.checkpoint import load_stage_checkpoint, save_stage_checkpoint
    from aeris_gb_b200.engine.optim import FlatOptimizer, OptimConfig
    from aeris_gb_b200.models.aeris import AerisConfig
    from aeris_gb_b200.models.stages import PipelineStage
    cfg = AerisConfig(img=(16, 32), window=(8, 8), in_channels=6, out_channels=3, dim=32, heads=2, head_dim=16,
                      mlp_dim=64, n_layers=2, sublayers=1, model_dtype=torch.float32)
    st = PipelineStage(cfg, range(0, 4))
    opt = FlatOptimizer(st, OptimConfig())
    d = tempfile.mkdtemp()
    files = save_stage_checkpoint(d, st, opt)
    before = {k: v.clone() for k, v in st.state_dict().items()}
    FaultInjector.corrupt_file(files[1], 4096)
    for p in st.parameters():
        p.data.add_(1.0)
    after_mod = {k: v.clone() for k, v in st.state_dict().items()}
    assert load_stage_checkpoint(d, st, opt, "cpu") is False
    for k, v in st.state_dict().items():
        assert torch.equal(v, after_mod[k]), "a failed load must leave the model untouched"
    # an intact directory restores exactly
    files = save_stage_checkpoint(d, st, opt)
    for p in st.parameters():
        p.data.mul_(0.0)
    assert load_stage_checkpoint(d, st, opt, "cpu") is True
    for k, v in st.state_dict().items():
        assert torch.equal(v, after_mod[k])
