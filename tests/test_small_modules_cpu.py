"""Small host-side modules: block sharding over the window-parallel grid, process-group bootstrap, the GIF script's
behaviour without its optional dependency."""
import importlib.util
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from aeris_gb_b200.data.sharding import gather_blocks, shard_block


def _gather_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    wp = (2, 2)
    g = torch.Generator().manual_seed(0)
    field = torch.randn(3, 8, 12, 5, generator=g)
    blk = shard_block(field, wp, (rank // wp[1], rank % wp[1]))
    assert blk.shape == (3, 4, 6, 5)
    full = gather_blocks(blk, wp)
    if rank == 0:
        torch.save(torch.equal(full, field), out)
    dist.barrier()
    dist.destroy_process_group()


def test_blocks_shard_and_gather_back_over_a_two_by_two_grid(tmp_path):
    from conftest import free_port
    out = str(tmp_path / "ok.pt")
    mp.spawn(_gather_worker, args=(4, free_port(), out), nprocs=4, join=True)
    assert torch.load(out) is True
    one = torch.arange(24.0).view(1, 2, 3, 4)
    assert torch.equal(gather_blocks(shard_block(one, (1, 1), (0, 0)), (1, 1)), one)


def test_single_process_bootstrap_without_a_launcher(monkeypatch):
    from aeris_gb_b200.utils.dist_setup import setup, teardown
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        monkeypatch.delenv(k, raising=False)
    monkeypatch.setenv("CUDA_VISIBLE_DEVICES", "")
    rank, world, device = setup()
    assert (rank, world) == (0, 1) and device.type in ("cpu", "cuda")
    teardown()


@pytest.mark.skipif(importlib.util.find_spec("matplotlib") is not None, reason="matplotlib is installed")
def test_gif_script_names_its_missing_dependency(tmp_path):
    import numpy as np
    from aeris_gb_b200.cli import animate
    np.save(tmp_path / "r.npy", np.zeros((2, 69, 4, 8), dtype=np.float32))
    with pytest.raises(SystemExit, match="matplotlib"):
        animate.main(["--input", str(tmp_path / "r.npy"), "--out", str(tmp_path / "o.gif")])
