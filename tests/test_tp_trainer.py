"""Tensor-parallel MLP inside the product: Trainer-level parity with the replicated model, shared clipping norm and the
checkpoint round trip (full tensors on disk), on gloo ranks here and on two GPUs over the fused kernels."""
import os
import subprocess
import sys

import pytest
import torch

WORKER = os.path.join(os.path.dirname(__file__), "tp_trainer_worker.py")


def _run(mode, port, tmp_path, env=None):
    e = dict(os.environ)
    e.update(env or {})
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", str(port), WORKER, mode, str(tmp_path / mode)],
                       capture_output=True, text=True, timeout=600, env=e)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]


@pytest.mark.parametrize("mode", ["sp", "wp"])
def test_tensor_parallel_trainer_matches_replicated_gloo(mode, tmp_path):
    _run(mode, 29621 + (mode == "wp"), tmp_path, {"CUDA_VISIBLE_DEVICES": ""})


@pytest.mark.gpu
@pytest.mark.parametrize("mode", ["sp", "wp"])
def test_tensor_parallel_trainer_matches_replicated_gpu(mode, tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    _run(mode, 29631 + (mode == "wp"), tmp_path)
