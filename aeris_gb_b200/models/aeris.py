"""AERIS pixel-level Swin diffusion transformer: stage modules with the reference's state-dict key layout.

Module / key parity with the reference (so per-stage checkpoints load unchanged):
  * input stage  ``proj.{weight,bias}``, ``latent_embed.w{1,2}.{weight,bias}``, ``ape.inv_freq``
    (src/aeris/models/parallel_swin.py:339-399)
  * Swin layer   ``modulelist.{j}.0.weight`` (RMSNorm), ``.1.norm.weight`` (unused, kept for key parity),
    ``.1.to_qkv.weight``, ``.1.wo.weight``, ``.2.weight``, ``.3.w1.weight``, ``.3.w2.weight``,
    ``.4.modulation.{0,2}.{weight,bias}`` (parallel_swin.py:401-472)
  * output stage ``norm.weight``, ``modulation.{0,2}.{weight,bias}``, ``head.weight`` (parallel_swin.py:490-532)
  * monolithic model ``input_stage.* / layers.{i}.* / output_stage.*`` and the per-stage -> monolithic conversion of
    src/aeris_wp_inference/model.py:431-495.

The modules operate on a *window-major token stream* (see :mod:`.layout`). On a CUDA device the blocks run on the
hand-written sm_100a kernels (:mod:`.fused`); on CPU they run the PyTorch oracle (:mod:`.oracle`).
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass, field

import torch
import torch.nn as nn
import torch.nn.functional as F
import torch.utils.checkpoint

from . import layout as LY
from . import oracle as O


@dataclass
class AerisConfig:
    img: tuple[int, int] = (720, 1440)
    window: tuple[int, int] = (60, 60)
    in_channels: int = 144          # noisy target + condition channels
    out_channels: int = 70
    dim: int = 1536
    heads: int = 12
    head_dim: int = 128
    mlp_dim: int = 6144
    n_layers: int = 8               # Swin layers (= PP_stages - 2 in the reference)
    sublayers: int = 3              # transformer blocks per layer
    layerwise_t_emb: bool = True
    after_mod_norm: bool = True     # modulate -> norm (True) or norm -> modulate (False)
    max_period: float = 10_000.0
    norm_eps: float | None = None   # None: machine epsilon of the block dtype (what nn.RMSNorm(eps=None) does)
    ape_row_offset: int | None = None  # None: 1 for 720-row grids (reference builds the APE on 721 rows, drops row 0)
    model_dtype: torch.dtype = torch.bfloat16
    data_dtype: torch.dtype = torch.float32
    wp: tuple[int, int] = (1, 1)
    sp: int = 1                     # Ulysses sequence-parallel degree
    # tensor-parallel MLP: w1 / w2 of every block split over ``tp`` ranks that hold different token rows of the same
    # sample (the SP group when sp > 1, else the WP group); ``tp_rank`` selects this rank's shard at construction
    tp: int = 1
    tp_rank: int = 0
    chunk_windows: int = 64
    shift_layers: str = "odd"       # which layers use the half-window shift: "odd" | "none"
    oracle_checkpoint: bool = False  # PyTorch (oracle) path only: recompute every block in backward
    use_rope: bool = False          # axial 2-D rotary embedding on q, k inside every window (the reference's is inert)
    rope_base: float = 10_000.0
    # model mode (parallel_swin.py:367-376, 394-397, 474-486): ``diffusion`` conditions every block on the noise level,
    # ``rit`` (random time interval) on an embedding of the forecast interval; with neither the blocks are plain
    # pre-norm transformer blocks and the model is a deterministic regressor
    diffusion: bool = True
    rit: bool = False
    emb_norm: bool = False          # rit: RMSNorm after the interval embedding

    @property
    def conditioned(self) -> bool:
        return self.diffusion or self.rit

    @property
    def n_blocks(self) -> int:
        return self.n_layers * self.sublayers

    def grid(self) -> LY.Grid:
        return LY.Grid(self.img[0], self.img[1], self.window[0], self.window[1], self.wp[0], self.wp[1], self.sp)

    def eps(self, dtype: torch.dtype) -> float:
        return self.norm_eps if self.norm_eps is not None else float(torch.finfo(dtype).eps)

    def layer_shift(self, i: int) -> tuple[int, int]:
        if self.shift_layers == "odd" and i % 2 == 1:
            return (self.window[0] // 2, self.window[1] // 2)
        return (0, 0)

    def param_count(self) -> int:
        d, hd, f = self.dim, self.heads * self.head_dim, self.mlp_dim
        mod = ((d * d + d if self.layerwise_t_emb else 0) + d * 6 * d + 6 * d) if self.conditioned else 0
        block = 2 * d + hd + 3 * hd * d + d * hd + 3 * d * f + mod
        inp = self.in_channels * d + d + 2 * (d * d + d)
        outp = d + (d * d + d if self.layerwise_t_emb else 0) + d * 2 * d + 2 * d + d * self.out_channels
        return block * self.n_blocks + inp + outp

    def flops_per_sample(self) -> float:
        return O.get_swin_flop_count(self.img, 1, self.n_blocks, self.in_channels, self.dim, self.mlp_dim, (1, 1),
                                     self.window)


class StreamContext:
    """Per-forward information the stage modules need about the token stream."""

    def __init__(self, cfg: AerisConfig, batch: int, rank: int = 0, peer_fn=None, wp_group=None, sp_group=None,
                 tp_group=None):
        self.cfg = cfg
        self.tp_group = tp_group      # tensor-parallel MLP group, None when TP = 1
        self.tp_exchange = None       # CUDA path: parallel.tensor.TPExchange of that group
        self.wp_group = wp_group      # torch.distributed group of the WP peers (CPU re-partition, result gathers)
        self.sp_group = sp_group      # Ulysses sequence-parallel group, None when SP = 1
        self.sp_exchange = None       # CUDA path: fused.SPExchange of that group
        self.grid = cfg.grid()
        self.batch = batch
        self.rank = rank
        self.peer_fn = peer_fn        # callable(tensor, direction) -> list of peer base addresses (WP) or None
        self._tables: dict = {}

    def rope(self, device):
        """(cos, sin) of the 2-D rotary embedding for one window, or None when the model does not use it."""
        if not self.cfg.use_rope:
            return None
        key = ("rope", str(device))
        if key not in self._tables:
            self._tables[key] = O.rope_2d_cache(self.cfg.window[0], self.cfg.window[1], self.cfg.head_dim,
                                                self.cfg.rope_base, device)
        return self._tables[key]

    def table(self, src_shift, dst_shift, device) -> torch.Tensor:
        key = (src_shift, dst_shift, str(device))
        if key not in self._tables:
            self._tables[key] = LY.gather_table(self.grid, src_shift, dst_shift, self.rank, self.batch).to(device)
        return self._tables[key]

    def regroup_unfused(self, x: torch.Tensor, src, dst) -> torch.Tensor:
        """Stand-alone re-partition between two window layouts (oracle path, and the final return to the plain
        layout before the output stage)."""
        if src == dst:
            return x
        fwd, bwd = self.table(src, dst, x.device), self.table(dst, src, x.device)
        if use_fused(x):
            from . import fused
            return fused.Regroup.apply(x, fwd, bwd, self.peer_fn)
        if self.grid.n_ranks == 1:
            _, row = LY.decode_table(fwd)
            return x[row.to(x.device)]
        return self.cpu_regroup(x, fwd, bwd)

    def cpu_regroup(self, x: torch.Tensor, table_fwd: torch.Tensor, table_bwd: torch.Tensor) -> torch.Tensor:
        """Multi-rank re-partition without peer memory (CPU / gloo runs): all-gather the WP ranks' rows, then index."""
        return _AllGatherRegroup.apply(x, table_fwd, table_bwd, self.wp_group)


class _AllGatherRegroup(torch.autograd.Function):
    @staticmethod
    def _run(x, table, group):
        import torch.distributed as dist
        world = dist.get_world_size(group)
        bufs = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(bufs, x.contiguous(), group=group)
        return LY.apply_gather_reference(table, bufs)

    @staticmethod
    def forward(ctx, x, table_fwd, table_bwd, group):
        ctx.table_bwd, ctx.group = table_bwd, group
        return _AllGatherRegroup._run(x, table_fwd, group)

    @staticmethod
    def backward(ctx, g):
        return _AllGatherRegroup._run(g.contiguous(), ctx.table_bwd, ctx.group), None, None, None


def use_fused(t: torch.Tensor) -> bool:
    return t.is_cuda and os.environ.get("AERIS_FORCE_ORACLE") != "1"


# ---------------------------------------------------------------------------------------------------- sub-modules
class LatentEmbedding(nn.Module):
    def __init__(self, dim):
        super().__init__()
        self.w1 = nn.Linear(dim, dim, bias=True)
        self.w2 = nn.Linear(dim, dim, bias=True)
        self.w1.is_time_emb = True
        self.w2.is_time_emb = True

    def forward(self, emb):
        return F.silu(self.w2(F.silu(self.w1(emb))))


class ApeBuffer(nn.Module):
    """Holds ``inv_freq`` for key parity; the encoding itself is produced by :func:`oracle.positional_encoding_2d`."""

    def __init__(self, channels, max_positions=10_000):
        super().__init__()
        ch = int(math.ceil(channels / 4) * 2)
        self.register_buffer("inv_freq", 1.0 / (max_positions ** (torch.arange(0, ch, 2).float() / ch)))


class AttentionParams(nn.Module):
    """``norm``: ``"unused"`` = present in the reference's diffusion checkpoints but never applied (kept frozen for
    key parity, parallel_swin.py:231-232, 265-266), ``"own"`` = the block's pre-norm in the plain mode, ``None`` = absent
    (rit)."""

    def __init__(self, dim, heads, head_dim, norm: str | None = "unused"):
        super().__init__()
        if norm is not None:
            self.norm = nn.RMSNorm(dim)
            if norm == "unused":
                self.norm.weight.requires_grad_(False)
        self.to_qkv = nn.Linear(dim, 3 * heads * head_dim, bias=False)
        self.wo = nn.Linear(heads * head_dim, dim, bias=False)


class FeedForwardParams(nn.Module):
    """``tp > 1``: this rank's shard of the SwiGLU weights (``w1``: its gate rows, then its up rows; ``w2``: its input
    columns). The full-size weights are drawn first and then cut, so that a tensor-parallel model built from the same
    seed holds exactly the slices of the unsharded model. The parameters carry ``tp_shard`` = "w1" / "w2"."""

    def __init__(self, dim, hidden, own_norm: bool = False, tp: int = 1, tp_rank: int = 0):
        super().__init__()
        if own_norm:                       # plain mode: the MLP normalises its own input (parallel_swin.py:88-96)
            self.norm = nn.RMSNorm(dim)
        self.w1 = nn.Linear(dim, 2 * hidden, bias=False)
        self.w2 = nn.Linear(hidden, dim, bias=False)
        if tp > 1:
            from ..parallel.tensor import shard_mlp_weights
            assert hidden % tp == 0
            w1_r, w2_r = shard_mlp_weights(self.w1.weight.detach(), self.w2.weight.detach(), tp, tp_rank)
            self.w1.weight, self.w1.out_features = nn.Parameter(w1_r), 2 * hidden // tp     # no further random draws
            self.w2.weight, self.w2.in_features = nn.Parameter(w2_r), hidden // tp
            self.w1.weight.tp_shard, self.w2.weight.tp_shard = "w1", "w2"


class ModulationLinear(nn.Module):
    def __init__(self, dim, out_dim, layerwise):
        super().__init__()
        if layerwise:
            self.modulation = nn.Sequential(nn.Linear(dim, dim, bias=True), nn.SiLU(), nn.Linear(dim, out_dim, bias=True))
        else:
            # same indices as the reference's two-element Sequential (SiLU at 0, Linear at 1)
            self.modulation = nn.Sequential(nn.SiLU(), nn.Linear(dim, out_dim, bias=True))

    def forward(self, x):
        return self.modulation(x)


# ---------------------------------------------------------------------------------------------------- stages
class InputStage(nn.Module):
    """fp32: (x + APE) -> Linear(in_channels -> dim) -> model dtype; sinusoidal noise-level embedding."""

    def __init__(self, cfg: AerisConfig):
        super().__init__()
        self.cfg = cfg
        self.proj = nn.Linear(cfg.in_channels, cfg.dim).to(cfg.data_dtype)
        self.proj.is_emb = True
        self.latent_embed = LatentEmbedding(cfg.dim).to(cfg.data_dtype)
        if cfg.rit and not cfg.diffusion:          # scalar forecast interval -> conditioning vector (:367-376)
            lin = nn.Linear(1, cfg.dim)
            lin.is_emb = lin.is_time_emb = True
            self.interval_embed = (nn.Sequential(lin, nn.RMSNorm(cfg.dim)) if cfg.emb_norm else lin).to(cfg.data_dtype)
        self.ape = ApeBuffer(cfg.in_channels)
        self._ape_tok: dict = {}

    def ape_tokens(self, ctx: StreamContext, device) -> torch.Tensor:
        key = (ctx.rank, str(device))
        if key not in self._ape_tok:
            cfg = self.cfg
            off = cfg.ape_row_offset if cfg.ape_row_offset is not None else (1 if cfg.img[0] == 720 else 0)
            pe = O.positional_encoding_2d(cfg.in_channels, cfg.img[0] + off, cfg.img[1], dtype=cfg.data_dtype)[off:]
            tok = LY.image_to_tokens(pe.unsqueeze(0), ctx.grid, (0, 0), ctx.rank)
            self._ape_tok[key] = tok.to(device)
        return self._ape_tok[key]

    def forward(self, x_tok: torch.Tensor, t: torch.Tensor, ctx: StreamContext):
        """x_tok: [B * tokens_per_rank, in_channels] fp32 in the unshifted layout; t: [B] noise level (radians)."""
        cfg = self.cfg
        ape = self.ape_tokens(ctx, x_tok.device)
        rows = ape.shape[0]
        B = x_tok.shape[0] // rows
        out = torch.empty((x_tok.shape[0], cfg.dim), dtype=cfg.model_dtype, device=x_tok.device)
        step = 1 << 16
        for b in range(B):
            for r in range(0, rows, step):
                sl = slice(b * rows + r, b * rows + min(rows, r + step))
                out[sl] = self.proj(x_tok[sl].to(cfg.data_dtype) + ape[r:r + step]).to(cfg.model_dtype)
        return out, self.noise_embedding(t)

    def noise_embedding(self, t: torch.Tensor | None) -> torch.Tensor:
        """Conditioning vector [B, dim]: the noise-level embedding (diffusion), the embedded forecast interval (rit,
        ``t`` = interval per sample), or zeros that nothing reads (plain mode)."""
        cfg = self.cfg
        if not cfg.diffusion:
            if cfg.rit:
                return self.interval_embed(t.reshape(-1, 1).to(cfg.data_dtype)).to(cfg.model_dtype)
            n = 1 if t is None else t.reshape(-1).shape[0]
            return torch.zeros((n, cfg.dim), dtype=cfg.model_dtype, device=self.proj.weight.device)
        emb = O.timestep_embedding(t.to(cfg.data_dtype), cfg.dim, cfg.max_period)
        if not cfg.layerwise_t_emb:
            emb = self.latent_embed(emb)
        return emb.to(cfg.model_dtype)

    def forward_images(self, x_img: torch.Tensor, c_img: torch.Tensor, cs: torch.Tensor, t: torch.Tensor, plan):
        """CUDA path from image-layout fields: x_img [B, hb, wb, C_out] (clean target when ``plan.noise``, else the
        noisy state), c_img [B, hb, wb, C_cond], cs [B, 2] = (cos t, sin t) (or (1, 0) when sampling). Noising,
        position encoding, window partition and the projection run in :mod:`.fused_io`."""
        from . import fused_io
        out = fused_io.EmbedFn.apply(x_img, c_img, cs, self.proj.weight, self.proj.bias, plan)
        return out, self.noise_embedding(t)


class SwinLayer(nn.Module):
    """``sublayers`` transformer blocks that share one window partition."""

    def __init__(self, cfg: AerisConfig):
        super().__init__()
        self.cfg = cfg
        d = cfg.dim
        if cfg.conditioned:
            self.modulelist = nn.ModuleList([
                nn.ModuleList([
                    nn.RMSNorm(d),
                    AttentionParams(d, cfg.heads, cfg.head_dim, None if cfg.rit else "unused"),
                    nn.RMSNorm(d),
                    FeedForwardParams(d, cfg.mlp_dim, tp=cfg.tp, tp_rank=cfg.tp_rank),
                    ModulationLinear(d, 6 * d, cfg.layerwise_t_emb),
                ]) for _ in range(cfg.sublayers)
            ])
        elif cfg.sublayers > 1:         # plain pre-norm blocks, module names as in parallel_swin.py:446-451
            self.modulelist = nn.ModuleList([
                nn.ModuleList([AttentionParams(d, cfg.heads, cfg.head_dim, "own"),
                               FeedForwardParams(d, cfg.mlp_dim, own_norm=True, tp=cfg.tp, tp_rank=cfg.tp_rank)])
                for _ in range(cfg.sublayers)])
        else:
            self.attn = AttentionParams(d, cfg.heads, cfg.head_dim, "own")
            self.ff = FeedForwardParams(d, cfg.mlp_dim, own_norm=True, tp=cfg.tp, tp_rank=cfg.tp_rank)

    def blocks(self):
        """(norm1 weight, attention parameters, norm2 weight, MLP parameters, modulation module or None) per block."""
        if self.cfg.conditioned:
            return [(n1.weight, attn, n2.weight, ff, mod) for n1, attn, n2, ff, mod in self.modulelist]
        pairs = list(self.modulelist) if self.cfg.sublayers > 1 else [(self.attn, self.ff)]
        return [(attn.norm.weight, attn, ff.norm.weight, ff, None) for attn, ff in pairs]

    def _plain_modulation(self, batch: int, device, dtype) -> torch.Tensor:
        """shift = scale = 0, gate = 1: the modulated block then IS the plain block x + f(norm(x))."""
        d = self.cfg.dim
        m = torch.zeros((batch, 6 * d), device=device, dtype=dtype)
        m[:, 2 * d:3 * d] = 1.0
        m[:, 5 * d:] = 1.0
        return m

    def forward(self, x: torch.Tensor, dt: torch.Tensor, ctx: StreamContext, regroup=None,
                publish_out: bool = False) -> torch.Tensor:
        """``regroup = (src_shift, dst_shift)``: the stream arrives in the ``src`` window layout and this layer works
        in ``dst``. On the CUDA path the re-partition (with its halo exchange under WP) is fused into the first
        block's modulate+norm kernel; the oracle path applies it as a separate gather. ``publish_out``: the caller
        re-partitions this layer's output next, so under WP the last block writes it into a peer-readable buffer."""
        cfg = self.cfg
        eps = cfg.eps(x.dtype)
        if regroup is not None and regroup[0] == regroup[1]:
            regroup = None
        blocks = self.blocks()
        # plain blocks normalise first (there is nothing to modulate before the norm)
        after_mod_norm = cfg.after_mod_norm and cfg.conditioned
        for j, (n1w, attn, n2w, ff, mod) in enumerate(blocks):
            if use_fused(x):
                from . import fused
                from ..ops import elementwise as E
                if ctx.grid.sp > 1 and ctx.sp_exchange is None:
                    raise RuntimeError("sequence parallelism on CUDA needs StreamContext.sp_exchange (fused.SPExchange)")
                m = fused.modulation(mod.modulation, dt) if mod is not None else \
                    self._plain_modulation(ctx.batch, x.device, torch.float32)
                meta = fused.BlockMeta(ctx.grid.windows_per_rank, ctx.grid.n_local, cfg.heads, cfg.head_dim,
                                       E.MODE_MOD_THEN_NORM if after_mod_norm else E.MODE_NORM_THEN_MOD,
                                       eps, cfg.chunk_windows, sp=ctx.sp_exchange if ctx.grid.sp > 1 else None,
                                       rope=ctx.rope(x.device), tp=ctx.tp_exchange if cfg.tp > 1 else None)
                if cfg.tp > 1 and ctx.tp_exchange is None:
                    raise RuntimeError("tensor parallelism on CUDA needs StreamContext.tp_exchange (tensor.TPExchange)")
                rg = None
                if j == 0 and regroup is not None:
                    rg = (ctx.table(regroup[0], regroup[1], x.device), ctx.table(regroup[1], regroup[0], x.device),
                          ctx.peer_fn)
                alloc = None
                if publish_out and j == len(blocks) - 1:
                    alloc = fused._pool_alloc(ctx.peer_fn)
                x = fused.FusedBlock.apply(x, m, meta, n1w, attn.to_qkv.weight, attn.wo.weight, n2w,
                                           ff.w1.weight, ff.w2.weight, rg, alloc)
            else:
                m = mod(dt.to(mod.modulation[-1].weight.dtype)) if mod is not None else \
                    self._plain_modulation(ctx.batch, x.device, x.dtype)
                if j == 0 and regroup is not None:
                    x = ctx.regroup_unfused(x, regroup[0], regroup[1])
                p = {"n1": n1w, "to_qkv": attn.to_qkv.weight, "wo": attn.wo.weight, "n2": n2w,
                     "w1": ff.w1.weight, "w2": ff.w2.weight}
                rope = ctx.rope(x.device)
                inner = (lambda q_, nw, nl, H, d: O.window_attention(q_, nw, nl, H, d, rope=rope)) if rope else None
                attn = inner
                if ctx.sp_group is not None and ctx.grid.sp > 1:
                    from ..parallel.sequence import sp_window_attention
                    attn = lambda qkv, nw, nl, H, d: sp_window_attention(qkv, nw, nl, H, d, ctx.sp_group,
                                                                           inner or O.window_attention)
                mlp = None
                if cfg.tp > 1:
                    from ..parallel.tensor import TPMlpCollective
                    mlp = lambda h2, w1=ff.w1.weight, w2=ff.w2.weight: TPMlpCollective.apply(h2, w1, w2, ctx.tp_group)
                run = lambda xx, mm: O.block_forward(xx, mm, p, n_win_per_sample=ctx.grid.windows_per_rank,
                                                     L=ctx.grid.n_local, heads=cfg.heads, head_dim=cfg.head_dim,
                                                     after_mod_norm=after_mod_norm, eps=eps, attention=attn, mlp=mlp)
                if cfg.oracle_checkpoint and torch.is_grad_enabled():
                    x = torch.utils.checkpoint.checkpoint(run, x, m, use_reentrant=False)
                else:
                    x = run(x, m)
        return x


class OutputStage(nn.Module):
    """fp32: RMSNorm -> modulate(shift, scale) -> Linear(dim -> out_channels, no bias)."""

    def __init__(self, cfg: AerisConfig):
        super().__init__()
        self.cfg = cfg
        d = cfg.dim
        self.norm = nn.RMSNorm(d).to(cfg.data_dtype)
        self.norm.is_head = True
        if cfg.conditioned:
            if cfg.layerwise_t_emb:
                self.modulation = nn.Sequential(nn.Linear(d, d, bias=True), nn.SiLU(), nn.Linear(d, 2 * d, bias=True))
            else:
                self.modulation = nn.Sequential(nn.SiLU(), nn.Linear(d, 2 * d, bias=True))
            self.modulation.to(cfg.data_dtype)
        self.head = nn.Linear(d, cfg.out_channels, bias=False).to(cfg.data_dtype)

    def forward_rows(self, x: torch.Tensor, shift: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
        cfg = self.cfg
        xf = x.to(cfg.data_dtype)
        xn = O.rms_norm(xf, self.norm.weight, cfg.eps(cfg.data_dtype))
        return self.head(xn * (1 + scale) + shift)

    def forward(self, x: torch.Tensor, dt: torch.Tensor, ctx: StreamContext) -> torch.Tensor:
        cfg = self.cfg
        if cfg.conditioned:
            shift, scale = self.modulation(dt.to(cfg.data_dtype)).chunk(2, dim=1)
        else:                               # plain mode: norm -> head (parallel_swin.py:526-528)
            shift = scale = torch.zeros((ctx.batch, cfg.dim), dtype=cfg.data_dtype, device=x.device)
        return _HeadFn.apply(x, shift, scale, self.norm.weight, self.head.weight, self)

    def loss_images(self, x, dt, x_img, cs, plan):
        """TrigFlow loss of the output stage straight from the stream (CUDA path; see :mod:`.fused_io`)."""
        from . import fused, fused_io
        shift, scale = fused.modulation(self.modulation, dt).chunk(2, dim=1)
        return fused_io.HeadLossFn.apply(x, shift, scale, self.norm.weight, self.head.weight, x_img, cs, plan)

    def predict_tokens(self, x, dt):
        """Network output in token order, fp32 ``[T, 128]`` (channels past ``out_channels`` are zero); no autograd."""
        from . import fused, fused_io
        with torch.no_grad():
            shift, scale = fused.modulation(self.modulation, dt).chunk(2, dim=1)
            return fused_io.head_forward(x, shift, scale, self.norm.weight, self.head.weight,
                                         self.cfg.eps(self.cfg.data_dtype))


class _HeadFn(torch.autograd.Function):
    """Output stage over a long token stream in 64k-row chunks. Only the (bf16) input is kept for the backward pass,
    which recomputes each chunk in fp32 and writes the input gradient chunk by chunk into one preallocated buffer,
    so no full-size fp32 copy of the stream ever exists."""
    STEP = 1 << 16

    @staticmethod
    def forward(ctx, x, shift, scale, norm_w, head_w, stage):
        B = shift.shape[0]
        rows = x.shape[0] // B
        out = torch.empty((x.shape[0], head_w.shape[0]), dtype=head_w.dtype, device=x.device)
        with torch.no_grad():
            for b in range(B):
                for r in range(0, rows, _HeadFn.STEP):
                    sl = slice(b * rows + r, b * rows + min(rows, r + _HeadFn.STEP))
                    out[sl] = stage.forward_rows(x[sl], shift[b:b + 1], scale[b:b + 1])
        ctx.stage = stage
        ctx.save_for_backward(x, shift, scale, norm_w, head_w)
        return out

    @staticmethod
    def backward(ctx, dout):
        x, shift, scale, norm_w, head_w = ctx.saved_tensors
        stage = ctx.stage
        B = shift.shape[0]
        rows = x.shape[0] // B
        dx = torch.empty_like(x)
        dshift, dscale = torch.zeros_like(shift), torch.zeros_like(scale)
        dnw, dhw = torch.zeros_like(norm_w), torch.zeros_like(head_w)
        for b in range(B):
            for r in range(0, rows, _HeadFn.STEP):
                sl = slice(b * rows + r, b * rows + min(rows, r + _HeadFn.STEP))
                with torch.enable_grad():
                    xc = x[sl].detach().requires_grad_(True)
                    sh = shift[b:b + 1].detach().requires_grad_(True)
                    sc = scale[b:b + 1].detach().requires_grad_(True)
                    y = stage.forward_rows(xc, sh, sc)
                    gx, gsh, gsc, gnw, ghw = torch.autograd.grad(y, (xc, sh, sc, stage.norm.weight, stage.head.weight),
                                                                 dout[sl])
                dx[sl] = gx
                dshift[b:b + 1] += gsh
                dscale[b:b + 1] += gsc
                dnw += gnw
                dhw += ghw
        return dx, dshift, dscale, dnw, dhw, None


# ---------------------------------------------------------------------------------------------------- full model
class AerisModel(nn.Module):
    """Input stage + ``n_layers`` Swin layers (odd ones on the half-window-shifted partition) + output stage."""

    def __init__(self, cfg: AerisConfig):
        super().__init__()
        self.cfg = cfg
        self.input_stage = InputStage(cfg)
        self.layers = nn.ModuleList([SwinLayer(cfg) for _ in range(cfg.n_layers)]).to(cfg.model_dtype)
        self.output_stage = OutputStage(cfg)

    def trunk(self, x: torch.Tensor, dt: torch.Tensor, ctx: StreamContext) -> torch.Tensor:
        cur = (0, 0)
        n = len(self.layers)
        for i, layer in enumerate(self.layers):
            nxt = self.cfg.layer_shift(i)
            after = self.cfg.layer_shift(i + 1) if i + 1 < n else (0, 0)     # layout of whoever consumes the output
            x = layer(x, dt, ctx, regroup=(cur, nxt), publish_out=(after != nxt))
            cur = nxt
        return ctx.regroup_unfused(x, cur, (0, 0))

    def forward_tokens(self, x_tok: torch.Tensor, t: torch.Tensor, ctx: StreamContext) -> torch.Tensor:
        x, dt = self.input_stage(x_tok, t, ctx)
        return self.output_stage(self.trunk(x, dt, ctx), dt, ctx)

    def loss_images(self, x_img, c_img, cs, t, ctx: StreamContext, plan) -> torch.Tensor:
        """Training loss from image-layout fields on the CUDA kernels end to end (noise drawn on the device from
        ``plan.seed``). Returns the sum over the local batch of the per-sample local-token-mean losses."""
        x, dt = self.input_stage.forward_images(x_img, c_img, cs, t, plan)
        return self.output_stage.loss_images(self.trunk(x, dt, ctx), dt, x_img, cs, plan)

    @torch.no_grad()
    def predict_images(self, x_img, c_img, t, ctx: StreamContext, plan) -> torch.Tensor:
        """One network evaluation for the sampler: ``x_img`` is the noisy state; returns F in token order [T, 128]."""
        cs = torch.tensor([[1.0, 0.0]], device=x_img.device).repeat(x_img.shape[0], 1)
        x, dt = self.input_stage.forward_images(x_img, c_img, cs, t, plan)
        return self.output_stage.predict_tokens(self.trunk(x, dt, ctx), dt)

    def forward(self, x_img: torch.Tensor, t: torch.Tensor) -> torch.Tensor:
        """x_img: [B, H, W, in_channels] fp32; t: [B]. Returns [B, H, W, out_channels] fp32 (single rank)."""
        B = x_img.shape[0]
        ctx = StreamContext(self.cfg, B)
        tok = LY.image_to_tokens(x_img, ctx.grid, (0, 0), 0)
        out = self.forward_tokens(tok, t, ctx)
        return LY.tokens_to_image([out], ctx.grid, (0, 0), B)


# ---------------------------------------------------------------------------------------------------- stage factory
def init_layer(stage_id: int, n_stages: int, cfg: AerisConfig) -> nn.Module:
    """Module for one pipeline stage: 0 = input stage, last = output stage, others one Swin layer
    (reference: ``init_layer`` parallel_swin.py:535-568)."""
    if stage_id == 0:
        return InputStage(cfg)
    if stage_id == n_stages - 1:
        return OutputStage(cfg)
    return SwinLayer(cfg).to(cfg.model_dtype)


def stage_to_model_key(stage_id: int, n_stages: int, key: str) -> str | None:
    """Maps a per-stage checkpoint key to the monolithic model key (src/aeris_wp_inference/model.py:479-495);
    returns None for the keys the reference drops (``latent_embed*`` of stage 0 when layerwise, ``*.1.norm*``)."""
    if stage_id == 0:
        return f"input_stage.{key}"
    if stage_id == n_stages - 1:
        return f"output_stage.{key}"
    return f"layers.{stage_id - 1}.{key}"
