"""Worker of the Trainer-level tensor-parallel test (gloo on CPU or NCCL on GPUs, 2 ranks): the same two training
steps with the MLP weights replicated and with them split over the tensor-parallel group must give the same losses
and, after gathering the shards, the same weights; a checkpoint written by the tensor-parallel run holds full
tensors and loads into both kinds of trainer.

usage: tp_trainer_worker.py <sp|wp> [checkpoint dir]"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from aeris_gb_b200.engine import checkpoint as CK  # noqa: E402
from aeris_gb_b200.engine.optim import OptimConfig  # noqa: E402
from aeris_gb_b200.engine.trainer import DiffusionConfig, Trainer  # noqa: E402
from aeris_gb_b200.models.aeris import AerisConfig  # noqa: E402
from aeris_gb_b200.parallel.tensor import full_state_dict  # noqa: E402


def rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12)).item()


def main():
    mode = sys.argv[1]
    ckpt_dir = sys.argv[2] if len(sys.argv) > 2 else None
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    cuda = torch.cuda.is_available()
    if cuda:
        torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
        dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
        dist.init_process_group("nccl", device_id=dev)
    else:
        dev = torch.device("cpu")
        dist.init_process_group("gloo")
    par = dict(wp=(1, 1), sp=world) if mode == "sp" else dict(wp=(1, world), sp=1)
    base = dict(img=(32, 64 * world), window=(16, 16), in_channels=10, out_channels=4, dim=256, heads=4, head_dim=64,
                mlp_dim=256 * world, n_layers=2, sublayers=1, norm_eps=1e-3, chunk_windows=3,
                model_dtype=torch.bfloat16 if cuda else torch.float32, **par)
    ocfg = OptimConfig(lr=1e-3, lr_rampup_img=0, grad_clip_max_norm=0.5)     # the clip is active: one shared norm
    dcfg = DiffusionConfig(cond_channels=6)
    grp = dist.group.WORLD
    kw = dict(wp_group=grp, sp_group=grp if mode == "sp" else None)
    plain = Trainer(AerisConfig(**base), ocfg, dcfg, dev, **kw)
    tens = Trainer(AerisConfig(**base, tp=world, tp_rank=rank), ocfg, dcfg, dev, **kw)
    g = torch.Generator().manual_seed(11 + rank)
    hb, wb = 32, 64 * world // par["wp"][1]
    losses = []
    for _ in range(2):
        x = torch.randn(2, hb, wb, 4, generator=g)
        c = torch.randn(2, hb, wb, 6, generator=g)
        if cuda:
            x, c = x.pin_memory(), c.pin_memory()
        losses.append((plain.train_step(x, c), tens.train_step(x, c)))
    tol = 3e-2 if cuda else 2e-4
    worst = max(abs(a - b) / max(abs(a), 1e-9) for a, b in losses)
    full = full_state_dict({k: v.detach() for k, v in tens.model.state_dict().items()}, grp)
    ref = plain.model.state_dict()
    for k, v in ref.items():
        if not v.dtype.is_floating_point or v.numel() <= 1:
            continue
        # bf16 runs: the first AdamW steps move every weight by about lr whatever the gradient's size, so a weight
        # whose gradient is rounding noise may move the other way; compare the tensors that are large against that
        if cuda and v.float().norm() < 20 * ocfg.lr * v.numel() ** 0.5:
            continue
        worst = max(worst, rel(full[k], v))
    ok = worst < tol and abs(plain.grad_norm() - tens.grad_norm()) <= tol * max(plain.grad_norm(), 1e-9)
    if ckpt_dir:
        CK.save_stage_checkpoint(ckpt_dir, tens.model, tens.opt, write=rank == 0)
        dist.barrier()
        for cfg_kw, label in ((dict(), "plain"), (dict(tp=world, tp_rank=rank), "tp")):
            fresh = Trainer(AerisConfig(**base, **cfg_kw), ocfg, dcfg, dev, seed=99, **kw)
            assert CK.load_stage_checkpoint(ckpt_dir, fresh.model, fresh.opt, dev), label
            a = dict(fresh.opt.master_state_dict())       # full tensors from either kind of optimizer
            b = dict(tens.opt.master_state_dict())
            for k in b:
                ok = ok and rel(a[k].to(b[k].device), b[k]) < 1e-6
            ok = ok and fresh.opt.cur_nimg == tens.opt.cur_nimg and fresh.opt.step_count == tens.opt.step_count
    if cuda:
        from aeris_gb_b200.ops import lib as L
        L.check_status()
    print(f"rank {rank}: mode {mode} losses {losses} worst {worst:.3e} ok {ok}", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
