"""Pipeline-parallel ensemble inference engine: forward-only fill/drain over the ensemble members.

Counterpart of the reference's ``InferenceEngine`` (src/aeris/parallelism/sp_inference_engine.py:104-656): same rank
grid as training, members as micro-batches, no-grad forward, the last stage returns every result to stage 0
(``SendResult`` / ``ReturnResult``, :200-233, :522-525). One call of :meth:`exec_schedule` is one network evaluation
for all members; the TrigFlow sampler drives it from the first stage (see ``cli/pp_generate.py``). Differences: sends
are non-blocking with the waits deferred (the reference puts a barrier between the activation and the embedding),
results are not gathered over SP through a sleep-guarded ``gather`` but concatenated by the caller when needed.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..parallel import schedule as SCH
from .pipeline import EngineConfig, ParallelEngine


class InferenceEngine(ParallelEngine):
    def __init__(self, *a, members: int = 1, **kw):
        ecfg: EngineConfig = a[3] if len(a) > 3 else kw["ecfg"]
        ecfg.gas = members
        super().__init__(*a, **kw)
        self.members = members
        # forward only: the fp32 masters, gradient accumulators, Adam moments and EMA that the training engine set up
        # for the bf16 parameters (16 to 20 bytes per parameter) are released; the parameters keep viewing the flat
        # bf16 buffer, the fp32 ends keep their (small) master buffer because they view it
        for seg in getattr(self.opt, "segments", []):
            if getattr(seg, "low_precision", False) and getattr(seg, "model_flat", None) is not None:
                for prm in seg.params:
                    if hasattr(prm, "main_grad"):
                        del prm.main_grad
                seg.master = seg.grad = seg.m = seg.v = seg.ema = None
        self.schedule = SCH.EnsembleInferenceSchedule(members, self.PP, self.c.pp)
        nb = self.schedule.num_pipe_buffers()
        self.buf = {k: [None] * nb for k in self.buf}
        self.module.eval()
        self.results: list[torch.Tensor | None] = [None] * members
        self._model_in = None
        self._t = None
        self._mb = 0
        self._ret = 0
        self.first_rank = self.grid.rank_of(self.c.dp, self.c.wp_y, self.c.wp_x, 0, self.c.sp)
        self.last_rank = self.grid.rank_of(self.c.dp, self.c.wp_y, self.c.wp_x, self.PP - 1, self.c.sp)
        if self.PP > 1:
            self.links.peer["result"] = self.last_rank if self.is_first_stage() else self.first_rank
        self._imap.update({SCH.SendResult: self.send_result, SCH.ReturnResult: self.return_result})

    def load_checkpoint(self, load_ema: bool = True, prefix: str = "") -> bool:
        """Weights only, the EMA copy by default (sp_inference_engine.py:552-573). ``prefix``: in front of the file
        names, e.g. ``it_5000_`` for a numbered copy."""
        from .checkpoint import load_stage_weights
        ok = load_stage_weights(self.ecfg.checkpoint_dir, self.module, use_ema=load_ema, prefix=prefix)
        if dist.is_initialized():
            dist.barrier()
        return ok

    def load(self, buffer_id):
        """Micro-batch = member: the caller's model input rows for member ``_mb`` and the shared noise level."""
        self.buf["inputs"][buffer_id] = self._model_in[self._mb]
        self.buf["t"][buffer_id] = self._t
        self._mb += 1

    def fwd(self, buffer_id):
        with torch.no_grad():
            x = self.buf["inputs"][buffer_id]
            if self.is_first_stage():
                y, dt = self.module(x, None, self.buf["t"][buffer_id], self.ctx)
            else:
                y, dt = self.module(x, self.buf["dt_in"][buffer_id], None, self.ctx)
        self.buf["outputs"][buffer_id], self.buf["dt_out"][buffer_id] = y, dt

    def process_recv(self, buffer_id):
        works, x, dt = self._pending.pop(("act", buffer_id))
        self.links.wait(works)
        self.buf["inputs"][buffer_id], self.buf["dt_in"][buffer_id] = x, dt

    def send_result(self, buffer_id):
        y = self.buf["outputs"][buffer_id]
        if self.PP == 1:
            self._local_result = y
            return
        self.links.send("result", [y.float()])

    def return_result(self, buffer_id):
        if self.PP == 1:
            out = self._local_result
        else:
            out = torch.empty((self.tokens, self.cfg.out_channels), dtype=torch.float32, device=self.device)
            self.links.wait(self.links.post_recv("result", [out]))
        self.results[self._ret] = out
        self._ret += 1

    def exec_schedule(self, model_in: list[torch.Tensor] | None = None, t: torch.Tensor | None = None):
        """One network evaluation for every member. ``model_in``: per-member rows [tokens, C_in] (first stage only);
        ``t``: [1] noise level. Returns the per-member outputs on the first stage (None elsewhere)."""
        self._model_in, self._t, self._mb, self._ret = model_in, t, 0, 0
        if not self.is_first_stage() and t is None:
            pass
        for cmds in self.schedule:
            for cmd in cmds:
                self._imap[type(cmd)](**cmd.kwargs)
        self._wait_sends()
        self.check_device()
        return self.results if self.is_first_stage() else None
