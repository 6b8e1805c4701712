"""Worker of the tensor-parallel MLP test: the fused all-gather -> GEMM and GEMM -> reduce-scatter kernels against the
unsharded MLP computed in fp32 PyTorch from the same full weights, forward and backward."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from aeris_gb_b200.ops import lib as L  # noqa: E402
from aeris_gb_b200.parallel import tensor as TP  # noqa: E402


def rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12)).item()


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=dev)
    D, F, n_loc = 512, 1024, 1000          # n_loc is not a multiple of any tile size on purpose
    g = torch.Generator().manual_seed(5)
    w1 = (torch.randn(2 * F, D, generator=g) * D ** -0.5).to(dev).bfloat16()
    w2 = (torch.randn(D, F, generator=g) * F ** -0.5).to(dev).bfloat16()
    x_full = torch.randn(world * n_loc, D, generator=g).to(dev).bfloat16()
    dy_full = torch.randn(world * n_loc, D, generator=g).to(dev).bfloat16()
    sl = slice(rank * n_loc, (rank + 1) * n_loc)
    w1_r, w2_r = TP.shard_mlp_weights(w1, w2, world, rank)
    w1_r.requires_grad_(True)
    w2_r.requires_grad_(True)
    tpx = TP.TPExchange(dist.group.WORLD, dev)
    worst = {}
    for it in range(2):                     # twice: buffers, counters and barrier epochs are reused
        h = x_full[sl].clone().requires_grad_(True)
        y = TP.TPMlpFn.apply(h, w1_r, w2_r, tpx)
        y.backward(dy_full[sl])
        # unsharded reference in fp32
        xr = x_full.float().requires_grad_(True)
        w1f, w2f = w1.float().requires_grad_(True), w2.float().requires_grad_(True)
        u = xr @ w1f.t()
        yr = (torch.nn.functional.silu(u[:, :F]) * u[:, F:]) @ w2f.t()
        yr.backward(dy_full.float())
        g1_r, g2_r = TP.shard_mlp_weights(w1f.grad, w2f.grad, world, rank)
        errs = {"y": rel(y, yr[sl]), "dh": rel(h.grad, xr.grad[sl]), "dw1": rel(w1_r.grad, g1_r),
                "dw2": rel(w2_r.grad, g2_r), "y_vs_nccl": rel(y, TP.tp_mlp_reference(x_full[sl], w1_r, w2_r,
                                                                                     dist.group.WORLD))}
        for k, v in errs.items():
            worst[k] = max(worst.get(k, 0.0), v)
        w1_r.grad = w2_r.grad = None
    L.check_status()
    ok = all(v < 2e-2 for v in worst.values())
    print(f"rank {rank}: {worst}", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
