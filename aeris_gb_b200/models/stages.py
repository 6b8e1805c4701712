"""Pipeline stages: the model is a chain of *logical* stages (input stage, one stage per Swin layer, output stage),
exactly the reference's PP layout (src/aeris/models/parallel_swin.py:563-568), and a *physical* pipeline rank runs a
contiguous run of them. Checkpoints are always written per logical stage, so they do not depend on the physical PP
degree and load into the reference's per-stage format.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from .aeris import AerisConfig, InputStage, OutputStage, StreamContext, SwinLayer, use_fused
from . import layout as LY


def split_stages(n_logical: int, n_physical: int) -> list[range]:
    """Contiguous, near-even assignment of logical stages to physical pipeline ranks. The two end stages are cheap,
    so the Swin layers are balanced first: with L layers and P ranks every rank gets L // P (+1 for the first
    L mod P ranks) layers, the input stage joins the first rank and the output stage the last."""
    L = n_logical - 2
    assert n_physical >= 1 and L >= n_physical or n_physical == n_logical, \
        f"cannot place {L} layers on {n_physical} pipeline ranks"
    if n_physical == n_logical:
        return [range(i, i + 1) for i in range(n_logical)]
    per, extra = divmod(L, n_physical)
    out, start = [], 1
    for p in range(n_physical):
        n = per + (1 if p < extra else 0)
        lo, hi = start, start + n
        start = hi
        if p == 0:
            lo = 0
        if p == n_physical - 1:
            hi = n_logical
        out.append(range(lo, hi))
    return out


class PipelineStage(nn.Module):
    """The logical stages ``stage_ids`` of a model with ``cfg.n_layers + 2`` logical stages."""

    def __init__(self, cfg: AerisConfig, stage_ids: range):
        super().__init__()
        self.cfg = cfg
        self.stage_ids = list(stage_ids)
        self.n_logical = cfg.n_layers + 2
        self.has_input = 0 in self.stage_ids
        self.has_output = (self.n_logical - 1) in self.stage_ids
        self.input_stage = InputStage(cfg) if self.has_input else None
        self.layer_ids = [s - 1 for s in self.stage_ids if 0 < s < self.n_logical - 1]
        self.layers = nn.ModuleDict({str(i): SwinLayer(cfg).to(cfg.model_dtype) for i in self.layer_ids})
        self.output_stage = OutputStage(cfg) if self.has_output else None

    # layout the stream has when it ENTERS / LEAVES this physical stage
    def entry_shift(self):
        """The stream arrives in the layout the previous physical stage left it in: that of the layer just before
        this stage's first layer (plain after the input stage)."""
        if self.has_input:
            return (0, 0)
        first = self.layer_ids[0] if self.layer_ids else self.cfg.n_layers
        return self.cfg.layer_shift(first - 1) if first > 0 else (0, 0)

    def exit_shift(self):
        return (0, 0) if self.has_output or not self.layer_ids else self.cfg.layer_shift(self.layer_ids[-1])

    def _regroup(self, x, src, dst, ctx: StreamContext):
        return ctx.regroup_unfused(x, src, dst)

    def forward(self, x: torch.Tensor | None, dt: torch.Tensor | None, t: torch.Tensor | None, ctx: StreamContext,
                images=None, loss_io=None):
        """First stage: ``x`` = model input tokens [T, C_in] and ``t`` the noise levels; other stages: ``x`` = stream
        [T, D] in this stage's entry layout and ``dt`` the noise-level embedding. Returns ``(y, dt)``; on the last
        stage ``y`` is the prediction [T, C_out] in the plain layout.
        CUDA kernels at the ends: ``images = (x_img, c_img, cs, plan)`` replaces ``x`` on the first stage (noising,
        position encoding, window partition and projection in one pass), ``loss_io = (x_img, cs, plan)`` makes the
        last stage return the TrigFlow loss instead of the prediction (head, loss and its gradient fused)."""
        cur = self.entry_shift()
        if self.has_input:
            if images is not None:
                x_img, c_img, cs, plan = images
                x, dt = self.input_stage.forward_images(x_img, c_img, cs, t, plan)
            else:
                x, dt = self.input_stage(x, t, ctx)
            cur = (0, 0)
        for i in self.layer_ids:
            nxt = self.cfg.layer_shift(i)
            x = self.layers[str(i)](x, dt, ctx, regroup=(cur, nxt))
            cur = nxt
        if self.has_output:
            x = self._regroup(x, cur, (0, 0), ctx)
            if loss_io is not None:
                x = self.output_stage.loss_images(x, dt, *loss_io)
            else:
                x = self.output_stage(x, dt, ctx)
        return x, dt

    # ---- per-logical-stage state dicts (reference checkpoint layout) -------------------------------------------
    def logical_state_dicts(self, source: dict[str, torch.Tensor] | None = None) -> dict[int, dict]:
        sd = source if source is not None else self.state_dict()
        out: dict[int, dict] = {}
        for k, v in sd.items():
            if k.startswith("input_stage."):
                out.setdefault(0, {})[k[len("input_stage."):]] = v
            elif k.startswith("output_stage."):
                out.setdefault(self.n_logical - 1, {})[k[len("output_stage."):]] = v
            elif k.startswith("layers."):
                _, idx, rest = k.split(".", 2)
                out.setdefault(int(idx) + 1, {})[rest] = v
        return out

    def key_for(self, logical_stage: int, key: str) -> str:
        if logical_stage == 0:
            return f"input_stage.{key}"
        if logical_stage == self.n_logical - 1:
            return f"output_stage.{key}"
        return f"layers.{logical_stage - 1}.{key}"
