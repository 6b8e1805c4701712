"""Window-parallel parity on 2 and 4 GPUs: the peer-memory halo gather must reproduce the single-GPU result."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n,sp", [(2, 1), (4, 1), (2, 2), (4, 2), (8, 1), (8, 2)])
def test_wp_parity(n, sp):
    """Window parallelism (halo pulled from peer memory) and Ulysses sequence parallelism (head<->sequence exchange
    fused into the QKV GEMM epilogue and the attention epilogues) against the single-GPU result."""
    if torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")
    worker = os.path.join(os.path.dirname(__file__), "wp_worker.py")
    port = 29500 + n + 10 * sp
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
                        "--master-addr", "127.0.0.1", "--master-port", str(port), worker, str(sp)],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]


@pytest.mark.parametrize("multicast", [0, 1])
def test_fused_gradient_reduce_adamw_allgather(multicast):
    n = 2
    if torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")
    worker = os.path.join(os.path.dirname(__file__), "fused_dp_worker.py")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
                        "--master-addr", "127.0.0.1", "--master-port", str(29520 + multicast), worker, str(multicast)],
                       capture_output=True, text=True, timeout=240)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]


@pytest.mark.parametrize("n", [2, 4])
def test_tensor_parallel_mlp(n):
    """All-gather -> GEMM (copier warps + arrival counters) and GEMM -> reduce-scatter (epilogue pushes) against the
    unsharded MLP, forward and backward."""
    if torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")
    worker = os.path.join(os.path.dirname(__file__), "tp_worker.py")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
                        "--master-addr", "127.0.0.1", "--master-port", str(29540 + n), worker],
                       capture_output=True, text=True, timeout=240)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]


@pytest.mark.parametrize("overlap", [0, 1])
def test_pipeline_parallel_nccl(overlap):
    """PP = 2 over NCCL p2p on the CUDA kernels against all stages on one GPU: plain 1F1B and the overlapped schedule
    (receives posted a step early on per-direction communicators). The worker's process group has a short time-out,
    so a transfer that never meets its counterpart ends the run with an error instead of waiting."""
    n = 2
    if torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")
    worker = os.path.join(os.path.dirname(__file__), "pp_worker.py")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
                        "--master-addr", "127.0.0.1", "--master-port", str(29560 + overlap), worker, str(overlap)],
                       capture_output=True, text=True, timeout=240)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]


@pytest.mark.parametrize("n,pp,wpx,sp,distopt", [(2, 2, 1, 1, 0), (2, 1, 2, 1, 0), (2, 1, 2, 1, 1)])
def test_pipeline_engine_with_fused_input_and_loss_kernels(n, pp, wpx, sp, distopt):
    """The pipeline engine with its end stages on the fused kernels (noising + position encoding + partition +
    projection; head + TrigFlow loss + gradient) and their counter-based noise, split over pipeline stages or window
    ranks, against the same engine on one GPU. ``distopt``: the split run steps with the sharded optimizer on the
    peer-memory kernels (gradient reduce-scatter + AdamW + weight all-gather)."""
    if torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")
    worker = os.path.join(os.path.dirname(__file__), "pp_worker.py")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
                        "--master-addr", "127.0.0.1", "--master-port", str(29590 + pp + 4 * distopt), worker, "1", str(pp),
                        str(wpx), str(sp), "1", str(distopt)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]


@pytest.mark.parametrize("n,pp,wpx,sp", [(4, 2, 2, 1), (4, 2, 1, 2), (8, 2, 2, 2)])
def test_pipeline_with_window_and_sequence_parallel_stages(n, pp, wpx, sp):
    """PP x WP x SP on GPUs (overlapped 1F1B over NCCL p2p; halo pulls and Ulysses pushes over peer memory inside every
    stage) against all stages on one GPU."""
    if torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")
    worker = os.path.join(os.path.dirname(__file__), "pp_worker.py")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
                        "--master-addr", "127.0.0.1", "--master-port", str(29570 + n + sp), worker, "1", str(pp), str(wpx),
                        str(sp)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
