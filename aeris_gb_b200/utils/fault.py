"""Failure detection and host-side fault injection.

The reference has only in-line checks: NaN asserts on pipeline sends and on the loss
(src/aeris/parallelism/parallel_engine.py:1020-1021, 1001-1003), a warm-up straggler alert (:1523-1533), a silent
``try/except`` around checkpoint load (:1143-1148) and job-level restart from periodic checkpoints. This module adds
what a production run on shared GPUs needs, without ever faulting a GPU:

  * :class:`Heartbeat` — every rank bumps a counter in the rendezvous store between steps; peers that stop beating are
    reported *before* the next collective is launched, so no kernel waits on a dead rank.
  * :class:`StepWatchdog` — flags steps slower than ``factor x`` the running median.
  * :func:`check_finite` — NaN/Inf guard on host-visible scalars (loss, gradient norm), raising ``NonFiniteError``.
  * :class:`FaultInjector` — host-side injection for tests: make a rank raise, skip its heartbeat, corrupt a
    checkpoint file, or poison a host tensor with NaN. Device-side injection (trapping or hanging a kernel) is
    deliberately not provided.
Device-side waits are bounded inside the kernels themselves (``csrc/common.cuh``); their time-outs surface through
``ops.lib.check_status``.
"""
from __future__ import annotations

import os
import statistics
import time

import torch


class RankFailure(RuntimeError):
    pass


class NonFiniteError(RuntimeError):
    pass


class Heartbeat:
    def __init__(self, store, rank: int, world: int, prefix: str = "hb", timeout_s: float = 30.0):
        self.store, self.rank, self.world, self.prefix, self.timeout_s = store, rank, world, prefix, timeout_s
        self._last_seen = {r: (0, time.monotonic()) for r in range(world)}
        self.count = 0

    def beat(self):
        self.count += 1
        self.store.set(f"{self.prefix}/{self.rank}", str(self.count))

    def mark_leaving(self):
        """A rank that leaves on purpose (between steps, nothing in flight) says so, so peers stop waiting for it."""
        self.store.set(f"{self.prefix}/{self.rank}", "-1")

    def _read(self, r: int) -> int:
        try:
            if hasattr(self.store, "check") and not self.store.check([f"{self.prefix}/{r}"]):
                return 0
            return int(self.store.get(f"{self.prefix}/{r}").decode())
        except Exception:
            return 0

    def dead_ranks(self) -> list[int]:
        now = time.monotonic()
        dead = []
        for r in range(self.world):
            if r == self.rank:
                continue
            v = self._read(r)
            if v == -1:
                dead.append(r)
                continue
            last_v, last_t = self._last_seen[r]
            if v != last_v:
                self._last_seen[r] = (v, now)
            elif now - last_t > self.timeout_s:
                dead.append(r)
        return dead

    def check(self):
        dead = self.dead_ranks()
        if dead:
            raise RankFailure(f"rank {self.rank}: no heartbeat from ranks {dead}")


class StepWatchdog:
    def __init__(self, factor: float = 3.0, warmup: int = 3):
        self.factor, self.warmup, self.times = factor, warmup, []

    def observe(self, seconds: float) -> bool:
        slow = False
        if len(self.times) >= self.warmup:
            slow = seconds > self.factor * statistics.median(self.times)
        self.times.append(seconds)
        self.times = self.times[-50:]
        return slow


def check_finite(name: str, value: float):
    if value != value or value in (float("inf"), float("-inf")):
        raise NonFiniteError(f"{name} is {value}")


class FaultInjector:
    """Host-side faults for tests, driven by the AERIS_FAULT environment variable, e.g.
    ``raise:rank=1:step=3``, ``silent:rank=2:step=1`` (stop beating), ``nan:rank=0:step=2``."""

    def __init__(self, spec: str | None = None):
        spec = spec if spec is not None else os.environ.get("AERIS_FAULT", "")
        self.kind, self.rank, self.step = None, None, None
        if spec:
            parts = spec.split(":")
            self.kind = parts[0]
            kv = dict(p.split("=") for p in parts[1:])
            self.rank, self.step = int(kv.get("rank", 0)), int(kv.get("step", 0))

    def fires(self, rank: int, step: int) -> bool:
        return self.kind is not None and rank == self.rank and step == self.step

    def maybe_raise(self, rank: int, step: int):
        if self.kind == "raise" and self.fires(rank, step):
            raise RuntimeError(f"injected failure on rank {rank} at step {step}")

    def silences(self, rank: int, step: int) -> bool:
        return self.kind == "silent" and rank == self.rank and step >= self.step

    def poison(self, t: torch.Tensor, rank: int, step: int) -> torch.Tensor:
        if self.kind == "nan" and self.fires(rank, step):
            t = t.clone()
            t.view(-1)[0] = float("nan")
        return t

    @staticmethod
    def corrupt_file(path: str, n_bytes: int = 64):
        with open(path, "r+b") as f:
            f.seek(max(0, os.path.getsize(path) // 2))
            f.write(os.urandom(n_bytes))
