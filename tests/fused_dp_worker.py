"""Worker of the multi-GPU test of the fused gradient reduce-scatter + AdamW + all-gather kernels: two identical
trainers take the same steps, one with NCCL all-reduce + the local fused AdamW, one with the peer-memory kernels; their
weights must agree. Run with and without the NVSwitch multicast path (argv[1] = 0/1)."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from aeris_gb_b200.engine.optim import OptimConfig  # noqa: E402
from aeris_gb_b200.engine.trainer import DiffusionConfig, Trainer, wp_grid_for  # noqa: E402
from aeris_gb_b200.models.aeris import AerisConfig  # noqa: E402
from aeris_gb_b200.ops import lib as L  # noqa: E402


def main():
    use_mc = bool(int(sys.argv[1])) if len(sys.argv) > 1 else False
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=dev)
    wp = wp_grid_for(world)
    cfg = AerisConfig(img=(64, 128), window=(16, 16), in_channels=12, out_channels=6, dim=128, heads=2, head_dim=64,
                      mlp_dim=256, n_layers=2, sublayers=1, norm_eps=1e-3, chunk_windows=3, wp=wp)
    ocfg = OptimConfig(lr=1e-3, lr_rampup_img=0, grad_clip_max_norm=0.05, weight_decay=0.1, decay_policy="all",
                       ema_halflife_img=50, ema_rampup_ratio=None)
    dcfg = DiffusionConfig(cond_channels=6)
    a = Trainer(cfg, ocfg, dcfg, dev, wp_group=dist.group.WORLD, fused_dp=False)
    b = Trainer(cfg, ocfg, dcfg, dev, wp_group=dist.group.WORLD, fused_dp=True, use_multicast=use_mc)
    hb, wb = 64 // wp[0], 128 // wp[1]
    g = torch.Generator().manual_seed(11 + rank)
    worst = 0.0
    for step in range(3):
        x = torch.randn(2, hb, wb, 6, generator=g).pin_memory()
        c = torch.randn(2, hb, wb, 6, generator=g).pin_memory()
        for t in (a, b):       # identical noise in both trainers
            t.rng.manual_seed(100 + step + rank)
            t.nl_rng.manual_seed(200 + step)
        la = a.train_step(x, c)
        lb = b.train_step(x, c)
        assert abs(la - lb) < 2e-2 * abs(la), (la, lb)
        na, nb = a.grad_norm(), b.grad_norm()
        assert abs(na - nb) < 2e-2 * na, (na, nb)
        for (n, p), (_, q) in zip(a.model.named_parameters(), b.model.named_parameters()):
            d = (p.float() - q.float()).abs().max().item()
            worst = max(worst, d / max(p.float().abs().max().item(), 1e-6))
    if not use_mc:
        # checkpoint round trip of the sharded optimizer: gathered into the per-stage file format by every rank, written
        # by rank 0, loaded into a differently initialised trainer; weights and the next step must agree
        import tempfile
        from aeris_gb_b200.engine.checkpoint import load_stage_checkpoint, save_stage_checkpoint
        box = [tempfile.mkdtemp() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        save_stage_checkpoint(box[0], b.model, b.opt, write=(rank == 0))
        dist.barrier()
        c = Trainer(cfg, ocfg, dcfg, dev, seed=999, wp_group=dist.group.WORLD, fused_dp=True, use_multicast=False)
        assert load_stage_checkpoint(box[0], c.model, c.opt, dev)
        c.seed, c.step_count = b.seed, b.step_count
        for (n, p), (_, q) in zip(b.model.named_parameters(), c.model.named_parameters()):
            assert torch.equal(p, q), n
        x = torch.randn(2, hb, wb, 6, generator=g).pin_memory()
        cc = torch.randn(2, hb, wb, 6, generator=g).pin_memory()
        for t in (b, c):
            t.nl_rng.manual_seed(777)
        lb, lc = b.train_step(x, cc), c.train_step(x, cc)
        assert abs(lb - lc) < 1e-4 * abs(lb), (lb, lc)
        for (n, p), (_, q) in zip(b.model.named_parameters(), c.model.named_parameters()):
            d = (p.float() - q.float()).abs().max().item()
            worst = max(worst, d / max(p.float().abs().max().item(), 1e-6))
    L.check_status()
    flag = torch.tensor([worst], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MAX)
    if rank == 0:
        print(f"fused_dp multicast={b.opt.uses_multicast} worst relative weight difference {flag.item():.2e}", flush=True)
    dist.destroy_process_group()
    sys.exit(0 if flag.item() < 2e-2 else 1)


if __name__ == "__main__":
    main()
