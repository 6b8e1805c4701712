"""Worker of the multi-GPU window-parallel parity test (one process per GPU, started by torch.distributed.run).

Every rank builds the same small model, runs it (a) on the whole image alone and (b) window-parallel on its own block
with the peer-memory halo gather, and compares outputs and all-reduced gradients. Exit code 0 = parity."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from aeris_gb_b200.engine.trainer import wp_grid_for  # noqa: E402
from aeris_gb_b200.models import layout as LY  # noqa: E402
from aeris_gb_b200.models.aeris import AerisConfig, AerisModel, StreamContext  # noqa: E402
from aeris_gb_b200.ops import lib as L  # noqa: E402
from aeris_gb_b200.parallel.symm import HaloExchange  # noqa: E402


def rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12)).item()


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=dev)
    sp = int(sys.argv[1]) if len(sys.argv) > 1 else 1
    wp = wp_grid_for(world // sp)
    base = dict(img=(64, 128), window=(16, 16), in_channels=12, out_channels=6, dim=256, heads=4, head_dim=64,
                mlp_dim=256, n_layers=3, sublayers=1, norm_eps=1e-3, chunk_windows=3)
    B = 2
    torch.manual_seed(7)
    ref = AerisModel(AerisConfig(**base)).to(dev)
    for n, p in ref.named_parameters():
        if "modulation" in n and p.dim() == 2:
            torch.nn.init.normal_(p, std=0.05)
    par = AerisModel(AerisConfig(**base, wp=wp, sp=sp)).to(dev)
    par.load_state_dict(ref.state_dict())
    g = torch.Generator(device="cpu").manual_seed(3)
    x = torch.randn(B, 64, 128, 12, generator=g).to(dev)
    r = torch.randn(B, 64, 128, 6, generator=g).to(dev)
    t = torch.tensor([0.4, 1.1], device=dev)
    # (a) single rank, whole image
    y_ref = ref(x, t)
    (y_ref * r).sum().backward()
    # (b) window parallel
    cfg = par.cfg
    grid = cfg.grid()
    halo = HaloExchange(dist.group.WORLD, dev)
    ctx = StreamContext(cfg, B, rank, halo.peer_fn)
    if sp > 1:
        from aeris_gb_b200.models.fused import SPExchange
        sp_group = None
        for r0 in range(0, world, sp):          # consecutive ranks form an SP group (sp is the fastest grid axis)
            g_ = dist.new_group(list(range(r0, r0 + sp)))
            if r0 <= rank < r0 + sp:
                sp_group = g_
        ctx.sp_group = sp_group
        ctx.sp_exchange = SPExchange(sp_group, dev)
    tok = LY.image_to_tokens(x, grid, (0, 0), rank)
    rt = LY.image_to_tokens(r, grid, (0, 0), rank)
    y = par.forward_tokens(tok, t, ctx)
    (y * rt).sum().backward()
    y_ref_tok = LY.image_to_tokens(y_ref.detach(), grid, (0, 0), rank)
    errs = {"out": rel(y.detach(), y_ref_tok)}
    for (n, p), (_, q) in zip(par.named_parameters(), ref.named_parameters()):
        if p.grad is None or q.grad is None or q.grad.float().norm() == 0:
            continue
        gsum = p.grad.float().clone()
        dist.all_reduce(gsum)
        errs[n] = rel(gsum, q.grad)
    L.check_status()
    worst = max(errs.values())
    flag = torch.tensor([worst], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MAX)
    if rank == 0:
        bad = {k: v for k, v in errs.items() if v > 3e-2}
        print(f"wp={wp} sp={sp} worst rel err {flag.item():.4f} out {errs['out']:.5f} bad={bad}", flush=True)
    dist.destroy_process_group()
    sys.exit(0 if flag.item() < 3e-2 else 1)


if __name__ == "__main__":
    main()
