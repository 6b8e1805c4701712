"""Process bootstrap from the torchrun environment (RANK / LOCAL_RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT).

The reference bootstraps through ``ezpz.setup_torch`` or raw MPI rank discovery (src/aeris/train.py:69,
src/aeris_wp_inference/inference.py:202-214); neither package exists here and neither is needed on one node."""
from __future__ import annotations

import os

import torch
import torch.distributed as dist


def setup(backend: str | None = None):
    """Returns (rank, world, device). Initialises torch.distributed when WORLD_SIZE > 1."""
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    cuda = torch.cuda.is_available()
    device = torch.device("cuda", local) if cuda else torch.device("cpu")
    if cuda:
        torch.cuda.set_device(device)
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        be = backend or ("nccl" if cuda else "gloo")
        if be == "nccl":
            dist.init_process_group(be, device_id=device)
        else:
            dist.init_process_group(be)
    return rank, world, device


def teardown():
    if dist.is_initialized():
        dist.destroy_process_group()
