"""ctypes binding of ``libaeris_b200.so`` (C ABI in ``csrc/api.h``).

The library is required on any machine that has a GPU: :func:`lib` raises if it cannot be loaded, so a GPU run can
never silently fall back to the PyTorch reference implementations. On a CPU-only machine the callers use the
pure-PyTorch oracle in :mod:`aeris_gb_b200.models.oracle` instead and never reach this module.
"""
from __future__ import annotations

import ctypes
import functools
import os

import torch

from .build import LIB_PATH, build, needs_build

_c_int = ctypes.c_int
_c_void_p = ctypes.c_void_p
_c_float = ctypes.c_float
_c_ll = ctypes.c_longlong


class KernelError(RuntimeError):
    pass


@functools.lru_cache(maxsize=None)
def lib() -> ctypes.CDLL:
    if needs_build() and os.environ.get("AERIS_NO_AUTOBUILD") != "1":
        build()
    if not LIB_PATH.exists():
        raise KernelError(f"native library missing: {LIB_PATH}; run `python -m aeris_gb_b200.ops.build`")
    return ctypes.CDLL(str(LIB_PATH))


def ptr(t: torch.Tensor | None) -> _c_void_p:
    return _c_void_p(0 if t is None else t.data_ptr())


def stream_ptr() -> _c_void_p:
    return _c_void_p(torch.cuda.current_stream().cuda_stream)


_STATUS: dict[int, torch.Tensor] = {}


def status_word() -> torch.Tensor:
    """Per-device int32 word that kernels set when a bounded wait runs out or a bounds check fails."""
    dev = torch.cuda.current_device()
    if dev not in _STATUS:
        _STATUS[dev] = torch.zeros(1, dtype=torch.int32, device=f"cuda:{dev}")
    return _STATUS[dev]


_ERR_NAMES = {
    1: "timeout waiting for a TMA-filled stage", 2: "timeout waiting for a free stage",
    3: "timeout waiting for an accumulator", 4: "timeout waiting for the epilogue to drain TMEM",
    5: "timeout waiting for a peer signal", 6: "bounds check failed", 7: "timeout inside the attention pipeline",
}


def check_status(sync: bool = True) -> None:
    """Synchronise and raise if any kernel recorded a device-side error since the last check."""
    w = status_word()
    if sync:
        torch.cuda.synchronize()
    code = int(w.item())
    if code != 0:
        w.zero_()
        raise KernelError(f"device-side error {code}: {_ERR_NAMES.get(code, 'unknown')}")


_LAUNCHES = 0


def launch_count() -> int:
    """Number of native kernel launches issued through this module since import."""
    return _LAUNCHES


def check(rc: int, what: str, kernels: int = 1) -> None:
    global _LAUNCHES
    _LAUNCHES += kernels
    if rc != 0:
        raise KernelError(f"{what} failed on the host side with code {rc}")
