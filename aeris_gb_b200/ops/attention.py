"""Python front end of the windowed flash attention kernels (``csrc/attention.cu``)."""
from __future__ import annotations

import math

import torch

from . import lib as _l


def _kernel_dim(d: int) -> int:
    """The kernels are built for 64- and 128-wide heads; other widths (for example 32) run zero-padded to the next one:
    zero columns change neither Q K^T nor the valid columns of P V."""
    if d in (64, 128):
        return d
    assert 0 < d < 128, f"head_dim {d} is not supported"
    return 64 if d < 64 else 128


def _pad_heads(t: torch.Tensor, parts: int, H: int, d: int, dp: int) -> torch.Tensor:
    T = t.shape[0]
    out = t.new_zeros((T, parts, H, dp))
    out[..., :d] = t.reshape(T, parts, H, d)
    return out.view(T, parts * H * dp)


def _unpad_heads(t: torch.Tensor, parts: int, H: int, d: int, dp: int) -> torch.Tensor:
    T = t.shape[0]
    return t.view(T, parts, H, dp)[..., :d].reshape(T, parts * H * d)


def attn_fwd(qkv: torch.Tensor, n_win: int, N: int, H: int, d: int, *, out: torch.Tensor | None = None,
             lse: torch.Tensor | None = None, scale: float | None = None) -> tuple[torch.Tensor, torch.Tensor]:
    """softmax(Q K^T * scale) V for every (window, head).

    ``qkv`` is ``[n_win * N, 3 * H * d]`` bf16 with columns ordered (q|k|v, head, d) and rows window-major.
    Returns ``(o [n_win * N, H * d] bf16, lse [n_win, H, N] fp32 in the log2 domain)``.
    """
    T, C = qkv.shape
    assert T == n_win * N and C == 3 * H * d and qkv.dtype == torch.bfloat16 and qkv.stride(1) == 1
    dp = _kernel_dim(d)
    if dp != d:
        o_p, lse = attn_fwd(_pad_heads(qkv, 3, H, d, dp), n_win, N, H, dp, lse=lse,
                            scale=scale if scale is not None else 1.0 / math.sqrt(d))
        o = _unpad_heads(o_p, 1, H, d, dp)
        if out is not None:
            out.copy_(o)
            o = out
        return o, lse
    if out is None:
        out = torch.empty((T, H * d), dtype=torch.bfloat16, device=qkv.device)
    if lse is None:
        lse = torch.empty((n_win, H, N), dtype=torch.float32, device=qkv.device)
    scale = scale if scale is not None else 1.0 / math.sqrt(d)
    ld = qkv.stride(0)
    rc = _l.lib().aeris_attn_fwd(_l.ptr(qkv), ld, 0, _l.ptr(qkv), ld, H * d, _l.ptr(qkv), ld, 2 * H * d,
                                 _l.ptr(out), out.stride(0), _l.ptr(lse), n_win, N, H, d,
                                 _l._c_float(scale), _l.ptr(_l.status_word()), _l.stream_ptr())
    _l.check(rc, "aeris_attn_fwd")
    return out, lse


def set_fwd_variant(poly: int = -1, mode: int = 0) -> None:
    """Variant of the forward kernel. ``poly`` (head_dim 64): -1 = scalar fp32 softmax arithmetic with every exponential
    on the exp unit; 0 = two-wide fp32 instructions; 2 = two-wide with two of every eight score pairs exponentiated by
    a cubic polynomial on the FMA pipe. ``mode``: 0 = probabilities through shared memory; 1 = probabilities kept in
    tensor memory as the A operand of P V; 2 = as 1 with four lighter CTAs per SM."""
    rc = _l.lib().aeris_attn_set_fwd_variant(int(poly), int(mode))
    if rc != 0:
        raise ValueError(f"no forward variant poly={poly} mode={mode}")


def attn_reference(qkv: torch.Tensor, n_win: int, N: int, H: int, d: int) -> torch.Tensor:
    """Plain PyTorch fp32 restatement (used by tests and by the CPU oracle)."""
    q, k, v = qkv.float().view(n_win, N, 3, H, d).permute(2, 0, 3, 1, 4)
    s = (q @ k.transpose(-1, -2)) / math.sqrt(d)
    o = s.softmax(-1) @ v
    return o.permute(0, 2, 1, 3).reshape(n_win * N, H * d)


def attn_bwd(qkv: torch.Tensor, o: torch.Tensor, d_o: torch.Tensor, lse: torch.Tensor, n_win: int, N: int, H: int,
             d: int, *, dqkv: torch.Tensor | None = None, delta: torch.Tensor | None = None,
             scale: float | None = None) -> torch.Tensor:
    """Gradient of :func:`attn_fwd` with respect to the fused qkv tensor (same layout as ``qkv``)."""
    T, C = qkv.shape
    assert o.shape == (T, H * d) and d_o.shape == (T, H * d) and d_o.stride(1) == 1 and o.stride(0) == d_o.stride(0)
    dp = _kernel_dim(d)
    if dp != d:
        g_p = attn_bwd(_pad_heads(qkv, 3, H, d, dp), _pad_heads(o, 1, H, d, dp), _pad_heads(d_o, 1, H, d, dp), lse,
                       n_win, N, H, dp, delta=delta, scale=scale if scale is not None else 1.0 / math.sqrt(d))
        g = _unpad_heads(g_p, 3, H, d, dp)
        if dqkv is not None:
            dqkv.copy_(g)
            g = dqkv
        return g
    if dqkv is None:
        dqkv = torch.empty_like(qkv)
    if delta is None:
        delta = torch.empty((n_win, H, N), dtype=torch.float32, device=qkv.device)
    scale = scale if scale is not None else 1.0 / math.sqrt(d)
    rc = _l.lib().aeris_attn_bwd(_l.ptr(qkv), qkv.stride(0), 0, H * d, 2 * H * d, _l.ptr(o), _l.ptr(d_o),
                                 o.stride(0), _l.ptr(lse), _l.ptr(delta), _l.ptr(dqkv), dqkv.stride(0), n_win, N, H,
                                 d, _l._c_float(scale), _l.ptr(_l.status_word()), _l.stream_ptr())
    _l.check(rc, "aeris_attn_bwd", kernels=2)
    return dqkv
