"""Observability: device-side timers (CUDA events, max over ranks), NVTX ranges, throughput in the reference's metric.

The reference accumulates host wall-clock per instruction without any device synchronisation, so it measures enqueue
time (src/aeris/parallelism/parallel_engine.py:1203-1223), and derives TFLOP/s/tile from its analytic FLOP model
(src/aeris/train.py:262-263, 288-296). Here a region is bracketed by CUDA events on the launching stream; times are
resolved lazily (no synchronisation inside the step) and reduced with MAX over ranks when reported.
"""
from __future__ import annotations

import contextlib
import time

import torch


class DeviceTimers:
    def __init__(self, enabled: bool = True, use_nvtx: bool = True):
        self.enabled = enabled
        self.use_nvtx = use_nvtx and torch.cuda.is_available()
        self._open: dict[str, list] = {}
        self._host: dict[str, float] = {}

    @contextlib.contextmanager
    def region(self, name: str):
        if not self.enabled:
            yield
            return
        cuda = torch.cuda.is_available()
        if self.use_nvtx:
            torch.cuda.nvtx.range_push(name)
        t0 = time.perf_counter()
        if cuda:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
        try:
            yield
        finally:
            if cuda:
                e1.record()
                self._open.setdefault(name, []).append((e0, e1))
            self._host[name] = self._host.get(name, 0.0) + time.perf_counter() - t0
            if self.use_nvtx:
                torch.cuda.nvtx.range_pop()

    def resolve(self, group=None, reset: bool = True) -> dict[str, float]:
        """Milliseconds per region since the last resolve (device time when CUDA is present, host time otherwise),
        MAX over the ranks of ``group`` when torch.distributed is initialised."""
        out = {}
        if torch.cuda.is_available() and self._open:
            torch.cuda.synchronize()
            for name, evs in self._open.items():
                out[name] = sum(a.elapsed_time(b) for a, b in evs)
        else:
            out = {k: v * 1e3 for k, v in self._host.items()}
        import torch.distributed as dist
        if dist.is_available() and dist.is_initialized() and out:
            names = sorted(out)
            dev = "cuda" if torch.cuda.is_available() and dist.get_backend(group) == "nccl" else "cpu"
            t = torch.tensor([out[n] for n in names], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
            out = dict(zip(names, t.tolist()))
        if reset:
            self._open.clear()
            self._host.clear()
        return out


class StepProfiler:
    """Optional ``torch.profiler`` capture of a window of training steps, exported as a Chrome trace (one file per
    rank). ``steps = (first, last)`` are absolute iteration numbers, ``last`` exclusive; ``None`` disables it. The
    kernels of this library appear under their own names; the NVTX ranges of :class:`DeviceTimers` nest around them."""

    def __init__(self, steps: tuple[int, int] | None, out_dir: str, rank: int = 0):
        self.steps, self.out_dir, self.rank = steps, out_dir, rank
        self._prof = None
        self.path = None

    def before_step(self, it: int) -> None:
        if self.steps is None or it != self.steps[0]:
            return
        from torch.profiler import ProfilerActivity, profile
        acts = [ProfilerActivity.CPU] + ([ProfilerActivity.CUDA] if torch.cuda.is_available() else [])
        self._prof = profile(activities=acts, record_shapes=False)
        self._prof.__enter__()

    def after_step(self, it: int) -> str | None:
        if self._prof is None or it + 1 < self.steps[1]:
            return None
        import os
        self._prof.__exit__(None, None, None)
        os.makedirs(self.out_dir, exist_ok=True)
        self.path = os.path.join(self.out_dir, f"trace_rank{self.rank}_it{self.steps[0]}-{self.steps[1]}.json")
        self._prof.export_chrome_trace(self.path)
        self._prof = None
        return self.path


def memory_report(device) -> str:
    """Peak allocated and reserved device memory in GB, as the reference prints in benchmark mode (train.py:293-299,
    where the reserved figure is mislabelled)."""
    if torch.device(device).type != "cuda":
        return ""
    return (f"alloc: {torch.cuda.max_memory_allocated(device) / 2 ** 30:.1f}GB, "
            f"res: {torch.cuda.max_memory_reserved(device) / 2 ** 30:.1f}GB")


def tflops_per_gpu(flops_per_sample: float, samples: int, seconds: float, world_size: int) -> float:
    """TFLOP/s per GPU in the reference's metric: analytic training FLOPs / step time / ranks (train.py:291)."""
    return flops_per_sample * samples / seconds / 1e12 / world_size


def wandb_payload(it: int, nimg: int, tflops: float, dt_iter: float, loss: float | None = None,
                  total_norm: float | None = None, lr: float | None = None, stage_norm: dict | None = None,
                  timers: dict | None = None, pp_rank: int = 0) -> dict:
    """Metric names as the reference logs them to wandb (train.py:311-348)."""
    d = {"train/iter": it, "train/nimg": nimg, "train/tflops_s_tile": tflops, "train/dt/iter": dt_iter}
    try:                                   # resident host memory of this process in GiB (train.py:316)
        import os

        import psutil
        d["train/mem/cpu"] = psutil.Process(os.getpid()).memory_info().rss / 2 ** 30
    except Exception:
        pass
    if loss is not None:
        d["train/loss"] = loss
    if total_norm is not None:
        d["train/total_norm"] = total_norm
    if lr is not None:
        d["lr"] = lr
    for k, v in (stage_norm or {}).items():
        d[f"train/stage_norm/stage_norm_{k}"] = v
    for k, v in (timers or {}).items():
        d[f"train/pp_timers/{k}/rank_{pp_rank}"] = v
    return d
