"""Reference arm: drives the UNMODIFIED modules of argonne-lcf/AERIS-GB (a plain copy of its ``src/`` tree under
``baseline/_ref``) on CUDA + NCCL with stock PyTorch kernels (cuBLAS, SDPA flash attention, torch.optim.AdamW).

Nothing of ``aeris_gb_b200`` is imported here and none of its kernels run: the arm is the comparison point for it.

What runs from the reference, unchanged:
  * training: ``ParallelSwinInputStage`` -> 40 x ``ParallelSwinLayer(sublayers=1)`` -> ``ParallelSwinOutputStage``
    (src/aeris/models/parallel_swin.py:339-532) with ``attn_fn="flash"``; every attention layer runs its four
    ``_SeqAllToAll`` exchanges (src/aeris/parallelism/sequence_parallel.py:89-142) over a one-rank NCCL group.
  * inference: the stages of ``LocalAERIS`` (src/aeris_wp_inference/model.py:327-477) with the attention function
    switched to the module's own ``optimized_attention`` (model.py:295).

What the reference's engine does around these modules needs >= 48 ranks, DeepSpeed, MPI and ``torch.xpu``
(src/aeris/parallelism/parallel_engine.py:72,706), so this file restates the minimum of it ("harness glue"):
  G1 window partition of the image into the ``[windows, tokens, C]`` layout with quadrant-major tokens
     (parallel_engine.py:183-199 with SP = 1), the 721-row position encoding and latitude weights
     (parallel_engine.py:611-639);
  G2 TrigFlow noise, model input and loss (parallel_engine.py:21-33, 673-678, 964-997);
  G3 the half-window shift of odd layers as one row permutation of the token stream (what ``torch.roll`` of the
     image does in model.py:101-114, and what the pipeline routing does in parallel_engine.py:335-373): one gather
     instead of un-partition + roll + partition, which is cheaper than either of the reference's ways;
  G4 activation checkpointing per layer and per chunk of windows (``torch.utils.checkpoint``): the reference has
     none and would need ~50 x the memory of a B200 at 1,036,800 tokens per GPU;
  G5 optimizer mode (a) (parallel_engine.py:702-741, 794-887, 1281-1319): flat fp32 gradient accumulator filled by
     per-parameter hooks, fp32 master weights, ``torch.optim.AdamW``, EMA, master -> bf16 copy, gradient
     ``all_reduce`` over the data-parallel ranks. The masters, optimizer and EMA stay on the GPU (the reference
     keeps them on the CPU), which only helps the reference;
  G6 the Heun sampler loop of src/aeris_wp_inference/inference.py:76-82,160-186 with the state kept on the device.
Data parallelism over N GPUs: one full sample per GPU, same global batch and tokens per GPU as the framework's
window-parallel run, no halo exchange.
"""
from __future__ import annotations

import math
import os
import sys
from types import SimpleNamespace

import torch
import torch.distributed as dist
import torch.nn.functional as F
from torch.utils.checkpoint import checkpoint

REF_ROOT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref")

# loss weights per variable for the 70-channel layout (parallel_engine.py:966-974)
_W_SURF = [0.1562, 0.0156, 0.0156, 0.0156]
_W_LEV = [0.0013, 0.0026, 0.0039, 0.0052, 0.0065, 0.0078, 0.0104, 0.0130, 0.0156, 0.0182, 0.0220, 0.0240, 0.0259]


def reference_available() -> str | None:
    """None when the copy of the reference's sources is in place, else the reason it is not."""
    need = [os.path.join(REF_ROOT, "aeris", "models", "parallel_swin.py"),
            os.path.join(REF_ROOT, "aeris", "parallelism", "sequence_parallel.py"),
            os.path.join(REF_ROOT, "aeris_wp_inference", "model.py")]
    missing = [p for p in need if not os.path.exists(p)]
    if missing:
        return "baseline/_ref lacks " + ", ".join(os.path.relpath(p, REF_ROOT) for p in missing) + \
            " (run python baseline/install_ref.py where the reference checkout is mounted)"
    return None


def _ref_modules():
    if REF_ROOT not in sys.path:
        sys.path.insert(0, REF_ROOT)
    from aeris.models import parallel_swin as SW          # noqa: E402  (reference code)
    from aeris_wp_inference import model as WPM           # noqa: E402  (reference code)
    return SW, WPM


# ---------------------------------------------------------------------------------------------------- layout (G1, G3)
class Layout:
    """Token order of the reference's training stages for SP = 1: ``[windows, (qy qx hy hx), C]``."""

    def __init__(self, H: int, W: int, ws: tuple[int, int], device):
        self.H, self.W, self.ws = H, W, ws
        self.nw = (H // ws[0]) * (W // ws[1])
        self.L = ws[0] * ws[1]
        pix = torch.arange(H * W, device=device).view(H, W)
        lay0 = self._partition(pix.unsqueeze(-1)).reshape(-1)
        lay1 = self._partition(torch.roll(pix, (-(ws[0] // 2), -(ws[1] // 2)), (0, 1)).unsqueeze(-1)).reshape(-1)
        inv0 = torch.empty_like(lay0); inv0[lay0] = torch.arange(H * W, device=device)
        inv1 = torch.empty_like(lay1); inv1[lay1] = torch.arange(H * W, device=device)
        self.pixel_of = lay0            # pixel id at every position of the unshifted layout
        self.up = inv0[lay1]            # shifted position -> unshifted position holding the same pixel
        self.down = inv1[lay0]

    def _partition(self, img: torch.Tensor) -> torch.Tensor:
        H, W, C = img.shape
        hy, hx = self.ws[0] // 2, self.ws[1] // 2
        x = img.view(H // self.ws[0], 2, hy, W // self.ws[1], 2, hx, C).permute(0, 3, 1, 4, 2, 5, 6)
        return x.reshape(self.nw, self.L, C)

    def partition(self, img: torch.Tensor) -> torch.Tensor:
        """[H, W, C] image -> [windows, tokens, C]."""
        return self._partition(img).contiguous()


class _Permute(torch.autograd.Function):
    """Rows of a ``[windows, tokens, D]`` stream re-ordered by a permutation; the gradient takes the inverse one."""

    @staticmethod
    def forward(ctx, x, perm, inv):
        ctx.inv = inv
        return x.reshape(-1, x.shape[-1]).index_select(0, perm).view_as(x)

    @staticmethod
    def backward(ctx, g):
        return g.reshape(-1, g.shape[-1]).index_select(0, ctx.inv).view_as(g), None, None


def _ape_image(SW_or_WPM, channels: int, H: int, W: int, device) -> torch.Tensor:
    """The reference's additive position encoding on its 721-row grid, first row dropped: [H, W, channels]."""
    ape = SW_or_WPM.PositionalEncoding2D(channels).to(device)
    rows = 721 if H == 720 else H + 1
    full = ape(torch.zeros(1, channels, rows, W, device=device))       # [1, C, rows, W]
    return full[0, :, 1:].permute(1, 2, 0).contiguous()


def _w_lat_image(H: int, W: int, add: float, device) -> torch.Tensor:
    rows = 721 if H == 720 else H + 1
    w = torch.cos(torch.deg2rad(torch.linspace(-90, 90, rows))) + add
    w = (w / w.mean())[1:]
    return w.view(H, 1, 1).expand(H, W, 1).to(device)


# ---------------------------------------------------------------------------------------------------- training arm
class ReferenceTrainer:
    """``train_step(target_host, cond_host) -> loss``: one optimizer step of the reference's modules on one full
    sample per GPU. ``dims``: dict(img, window, dim, heads, head_dim, mlp_dim, n_layers, in_ch, out_ch, chunk_windows)."""

    def __init__(self, dims: dict, device, group=None, seed: int = 1234, lr: float = 1e-3, ema: bool = True):
        SW, _ = _ref_modules()
        self.SW, self.d, self.dev, self.group = SW, dims, torch.device(device), group
        self.world = dist.get_world_size(group) if group is not None else 1
        self.rank = dist.get_rank(group) if group is not None else 0
        H, W = dims["img"]
        cfg = SimpleNamespace(model=SimpleNamespace(sinusoidal_emb_max_period=10_000,
                                                    layerwise_t_emb_after_mod_norm=True))
        torch.manual_seed(seed)
        kw = dict(diffusion=True, layerwise_t_emb=True)
        bf16, f32 = torch.bfloat16, torch.float32
        self.inp = SW.ParallelSwinInputStage(cfg, dims["in_ch"], dims["dim"], data_dtype=f32, model_dtype=bf16, **kw)
        self.layers = [SW.ParallelSwinLayer(cfg, dims["dim"], dims["heads"], dims["head_dim"], "pre", dims["mlp_dim"],
                                            tuple(dims["window"]), 10_000, bf16, "flash", sublayers=1, **kw)
                       for _ in range(dims["n_layers"])]
        self.out = SW.ParallelSwinOutputStage(cfg, dims["dim"], dims["out_ch"], "pre", data_dtype=f32, **kw)
        stages = [self.inp, *self.layers, self.out]
        # fp32 masters first (parallel_engine.py:137-139), the working copy is cast from them: bf16 layers, fp32 ends
        self.master = [p.detach().clone().to(self.dev, f32) for s in stages for p in s.parameters()]
        self.inp.to(self.dev, f32); self.out.to(self.dev, f32)
        for l in self.layers:
            l.to(self.dev, bf16)
        self.params = [p for s in stages for p in s.parameters()]
        # G5: flat fp32 accumulator, per-parameter views, hooks that add .grad into it and drop .grad
        n = sum(p.numel() for p in self.params)
        self.grad_bufs = torch.zeros(n, device=self.dev, dtype=f32)
        off = 0
        for p, m in zip(self.params, self.master):
            p.main_grad = self.grad_bufs[off:off + p.numel()].view(p.shape)
            m.grad = p.main_grad
            off += p.numel()
            p.register_post_accumulate_grad_hook(self._acc_hook)
        self.opt = torch.optim.AdamW(self.master, lr=lr, betas=(0.9, 0.999), weight_decay=0.01, eps=1e-8, fused=True)
        self.ema = [m.detach().clone() for m in self.master] if ema else None
        self.ema_halflife_img, self.cur_nimg = 500_000.0, 0
        # the sequence-parallel group of one rank: the stock _SeqAllToAll path runs its all_to_all_single on it
        self.sp_group = None
        if dist.is_initialized():
            for r in range(dist.get_world_size()):
                g = dist.new_group([r])
                if r == dist.get_rank():
                    self.sp_group = g
        self.lay = Layout(H, W, tuple(dims["window"]), self.dev)
        self.inp.ape_generated = self.lay.partition(_ape_image(SW, dims["in_ch"], H, W, self.dev))
        self.w_lat = self.lay.partition(_w_lat_image(H, W, 0.01, self.dev))
        w_var = torch.tensor(_W_SURF + _W_LEV * 5 + [0.0156], device=self.dev)
        self.w_var = (w_var if dims["out_ch"] == 70 else torch.full((dims["out_ch"],), 1.0 / dims["out_ch"],
                                                                      device=self.dev)).view(1, 1, -1)
        self.sigma_data, self.sigma_min, self.sigma_max = 1.0, 0.2, 500.0
        self.rng = torch.Generator(device=self.dev); self.rng.manual_seed(seed + 1000 + self.rank)
        self.nl_rng = torch.Generator(device=self.dev); self.nl_rng.manual_seed(seed + self.rank)
        self.param_count = n

    @staticmethod
    def _acc_hook(p):
        p.main_grad.add_(p.grad)
        p.grad = None

    # G2 (parallel_engine.py:21-33)
    def _noise(self, x):
        u = torch.rand([1, 1], device=self.dev, generator=self.nl_rng)
        tau = torch.exp(math.log(self.sigma_min) + u * (math.log(self.sigma_max) - math.log(self.sigma_min)))
        t = torch.atan(tau / self.sigma_data)
        z = torch.randn(x.shape, dtype=torch.float32, device=self.dev, generator=self.rng) * self.sigma_data
        return t, z

    def _run_layers(self, x, dt):
        cw = self.d["chunk_windows"]
        for i, layer in enumerate(self.layers):
            if i % 2 == 1:
                x = _Permute.apply(x, self.lay.up, self.lay.down)
            outs = [checkpoint(layer, xc, None, dt, self.sp_group, use_reentrant=False) for xc in x.split(cw, 0)]
            x = torch.cat(outs, 0)
            del outs
            if i % 2 == 1:
                x = _Permute.apply(x, self.lay.down, self.lay.up)
        return x

    def _head_loss(self, xc, dt, target, z, w_lat, cos_t, sin_t):
        out = self.out(xc, None, dt, self.sp_group)
        v_t = cos_t * z - sin_t * target
        return (w_lat * self.w_var * (self.sigma_data * out - v_t) ** 2).sum(dim=2).sum()

    def train_step(self, target_host: torch.Tensor, cond_host: torch.Tensor, marks=None) -> float:
        """target_host [1, H, W, out_ch], cond_host [1, H, W, cond_ch]: pinned fp32 host tensors. Returns the loss
        (a device -> host read). ``marks``: optional pair of CUDA events recorded after the input copy and before the
        loss read-back, for the device-only time of the step."""
        x_img = target_host.to(self.dev, non_blocking=True)[0]
        c_img = cond_host.to(self.dev, non_blocking=True)[0]
        if marks is not None:
            marks[0].record()
        x, cond = self.lay.partition(x_img), self.lay.partition(c_img)
        t, z = self._noise(x)
        cos_t, sin_t = torch.cos(t), torch.sin(t)
        inputs = torch.cat([(cos_t * x + sin_t * z) / self.sigma_data, cond], dim=-1)
        h, dt = self.inp(inputs, None, sigma_data=self.sigma_data, condition=None, auxilary=None, interval=t)
        h = self._run_layers(h, dt)
        cw = self.d["chunk_windows"]
        loss = 0.0
        for hc, xc, zc, wc in zip(h.split(cw, 0), x.split(cw, 0), z.split(cw, 0), self.w_lat.split(cw, 0)):
            loss = loss + checkpoint(self._head_loss, hc, dt, xc, zc, wc, cos_t, sin_t, use_reentrant=False)
        loss = loss / (self.lay.nw * self.lay.L)           # mean over tokens of the channel-summed error
        loss.backward()
        self._reduce_and_step()
        if marks is not None:
            marks[1].record()
        return float(loss.item())

    def _reduce_and_step(self):
        # parallel_engine.py:709-724 with GAS = 1
        if self.world > 1:
            dist.all_reduce(self.grad_bufs, group=self.group)
            self.grad_bufs.mul_(1.0 / self.world)
        total_norm = torch.norm(self.grad_bufs, p=2).item()
        clip = 1.0 / (total_norm + 1.0e-6)
        if clip < 1.0:
            self.grad_bufs.mul_(clip)
        self.total_norm = total_norm
        self.opt.step()                                   # master.grad are the views of grad_bufs
        with torch.no_grad():
            torch._foreach_copy_(self.params, self.master)    # parallel_engine.py:861-866
        self.cur_nimg += self.world
        if self.ema is not None:                          # parallel_engine.py:868-884
            half = min(self.ema_halflife_img, self.cur_nimg * 0.05)
            beta = 0.5 ** (self.world / max(half, 1e-8))
            torch._foreach_lerp_(self.ema, self.master, 1.0 - beta)
        self.grad_bufs.zero_()

    def flops_per_step(self, global_batch: int) -> float:
        d = self.d
        return self.SW.get_swin_flop_count(list(d["img"]), global_batch, d["n_layers"], d["in_ch"], d["dim"],
                                           d["mlp_dim"], [1, 1], list(d["window"]))


# ---------------------------------------------------------------------------------------------------- inference arm
class ReferenceForecaster:
    """One ensemble member per GPU on the stages of the reference's ``LocalAERIS``; ``step(state, forcing)`` advances
    the standardised state by one forecast step with the Heun sampler of inference.py:160-186."""

    def __init__(self, dims: dict, device, sampler_steps: int = 10, seed: int = 0):
        _, WPM = _ref_modules()
        self.d, self.dev = dims, torch.device(device)
        H, W = dims["img"]
        torch.manual_seed(1234)
        m = WPM.LocalAERIS(None, dims["heads"], dims["dim"], dims["head_dim"], dims["mlp_dim"], tuple(dims["window"]),
                           (H, W), 10_000, 1, 10_000, dims["n_layers"] + 2, dims["in_ch"], dims["out_ch"])
        self.model = m.to(self.dev).eval()
        for layer in m.layers:
            for sub in layer.modulelist:
                sub[1].attn_fn = sub[1].optimized_attention
        m.input_stage.ape_generated = _ape_image(WPM, dims["in_ch"], H, W, self.dev).view(1, H * W, dims["in_ch"])
        self.sigma_data, sigma_min, sigma_max, rho = 1.0, 0.2, 500.0, 10
        ramp = torch.linspace(0, 1, sampler_steps, device=self.dev)
        sig = (sigma_max ** (1 / rho) + ramp * (sigma_min ** (1 / rho) - sigma_max ** (1 / rho))) ** rho
        t = torch.atan(sig / self.sigma_data)
        self.t_steps = torch.cat([t, torch.zeros_like(t[:1])])
        self.n = sampler_steps
        self.gen = torch.Generator(device=self.dev); self.gen.manual_seed(seed)
        self.evals = 0

    def _shift(self, x, up: bool):
        H, W = self.d["img"]
        h, w = self.d["window"][0] // 2, self.d["window"][1] // 2
        img = x.view(1, H, W, -1)
        return torch.roll(img, shifts=(-h, -w) if up else (h, w), dims=(1, 2)).reshape(1, H * W, -1)

    @torch.no_grad()
    def model_eval(self, model_in, s):
        """``LocalAERIS.forward`` (model.py:468-477) with the one-rank shift done in place of ``swin_shift``."""
        m = self.model
        out, t = m.input_stage(model_in, s)
        for i, layer in enumerate(m.layers):
            if i % 2 == 1:
                out = self._shift(out, True)
            out = layer(out, t)
            if i % 2 == 1:
                out = self._shift(out, False)
        self.evals += 1
        return m.output_stage(out, t)

    @torch.no_grad()
    def step(self, state: torch.Tensor, forcing: torch.Tensor) -> torch.Tensor:
        """state [1, H*W, out_ch], forcing [1, H*W, in_ch - 2 out_ch] on the device (standardised, unit statistics)."""
        sd = self.sigma_data
        cond = torch.cat([state, forcing], dim=2)
        x_t = torch.randn(state.shape, generator=self.gen, device=self.dev) * sd
        for k in range(self.n):
            s, t = self.t_steps[k], self.t_steps[k + 1]
            delta = t - s
            F_s = self.model_eval(torch.cat([x_t / sd, cond], dim=2), s.view(1))
            x_e = x_t + delta * sd * F_s
            if k < self.n - 1:
                F_t = self.model_eval(torch.cat([x_e / sd, cond], dim=2), t.view(1))
                x_t = x_t + delta * sd * 0.5 * (F_s + F_t)
            else:
                x_t = x_e
        return state + x_t                                  # unit statistics: residual added in standardised space
