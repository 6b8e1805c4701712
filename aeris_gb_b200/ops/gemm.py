"""Python front end of the tcgen05 GEMM (``csrc/gemm.cu``)."""
from __future__ import annotations

import os

import torch

from . import lib as _l

# The two-CTA (cta_group::2, 256 x 256 tile per SM pair) kernel is used for every product whose N is a multiple of 256
# unless AERIS_GEMM_2CTA=0.
TWO_CTA_DEFAULT = os.environ.get("AERIS_GEMM_2CTA", "1") != "0"

EPI_STORE, EPI_SWIGLU, EPI_GATE_RESID, EPI_ACC_F32, EPI_STORE_F32, EPI_SWIGLU_BOTH, EPI_SWIGLU_BWD = range(7)


def _ld(t: torch.Tensor) -> int:
    assert t.dim() == 2 and t.stride(1) == 1, "operands must be row-major 2-D views"
    return t.stride(0)


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_t: bool = False, b_t: bool = False, out: torch.Tensor | None = None,
         epi: int = EPI_STORE, resid: torch.Tensor | None = None, gate: torch.Tensor | None = None,
         rows_per_gate: int = 0, aux: torch.Tensor | None = None, k_splits: int = 1, bn: int = 0,
         two_cta: bool | None = None) -> torch.Tensor:
    """``out (op)= A @ B^T`` on the tensor cores.

    ``a`` is ``[M, K]`` (or, with ``a_t``, the stored tensor is ``[K, M]`` and is used transposed); ``b`` is
    ``[N, K]`` (with ``b_t``: stored ``[K, N]``). All operands bf16, fp32 accumulation.

    epi: EPI_STORE bf16 out; EPI_SWIGLU ``silu(acc[:, :F]) * acc[:, F:]`` (b = [2F, K]) -> ``[M, F]``;
    EPI_GATE_RESID ``resid + gate * acc`` (gate fp32 ``[M // rows_per_gate, N]``; ``aux`` optionally receives the
    raw product); EPI_ACC_F32 ``out += acc`` in fp32 (split-K allowed); EPI_STORE_F32 fp32 out;
    EPI_SWIGLU_BOTH = EPI_SWIGLU that also writes the raw ``[gate | up]`` product to ``aux [M, 2F]``;
    EPI_SWIGLU_BWD: the product is d(act) ``[M, F]``, ``resid`` holds ``u = [gate | up]`` and ``out`` receives d(u).
    """
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
    if a_t:
        K, M = a.shape
    else:
        M, K = a.shape
    if b_t:
        Kb, N = b.shape
    else:
        N, Kb = b.shape
    assert K == Kb, (a.shape, b.shape, a_t, b_t)
    swiglu_f = 0
    n_out = N
    if epi in (EPI_SWIGLU, EPI_SWIGLU_BOTH):
        assert N % 2 == 0 and not b_t
        swiglu_f = N // 2
        n_out = swiglu_f
        assert epi == EPI_SWIGLU or (aux is not None and aux.shape == (M, N))
    if epi == EPI_SWIGLU_BWD:
        # acc = d(act) [M, F]; resid = u [M, 2F]; out = d(u) [M, 2F] (may alias resid)
        assert resid is not None and out is not None and resid.shape == (M, 2 * N) and out.shape == (M, 2 * N)
        swiglu_f = N
    if out is None:
        dt = torch.float32 if epi in (EPI_ACC_F32, EPI_STORE_F32) else torch.bfloat16
        out = (torch.zeros if epi == EPI_ACC_F32 else torch.empty)((M, n_out), dtype=dt, device=a.device)
    assert out.shape == (M, n_out) or epi == EPI_SWIGLU_BWD
    if two_cta is None:
        two_cta = TWO_CTA_DEFAULT and bn == 0
    if two_cta and N % 256 == 0:
        rc = _l.lib().aeris_gemm_bf16_2cta(
            _l.ptr(a), _l.ptr(b), _l.ptr(out), M, N, K, _ld(a), _ld(b), _ld(out), int(a_t), int(b_t), epi,
            _l.ptr(resid), _ld(resid) if resid is not None else 0, _l.ptr(gate), rows_per_gate,
            _l.ptr(aux), _ld(aux) if aux is not None else 0, swiglu_f, k_splits, _l.ptr(_l.status_word()),
            _l.stream_ptr())
        _l.check(rc, "aeris_gemm_bf16_2cta")
        return out
    if bn == 0:
        bn = 256 if N % 256 == 0 else 128
    rc = _l.lib().aeris_gemm_bf16(
        _l.ptr(a), _l.ptr(b), _l.ptr(out), M, N, K, _ld(a), _ld(b), _ld(out), int(a_t), int(b_t), epi,
        _l.ptr(resid), _ld(resid) if resid is not None else 0, _l.ptr(gate), rows_per_gate,
        _l.ptr(aux), _ld(aux) if aux is not None else 0, swiglu_f, k_splits, bn, _l.ptr(_l.status_word()),
        _l.stream_ptr())
    _l.check(rc, "aeris_gemm_bf16")
    return out
