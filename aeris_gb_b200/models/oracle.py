"""Pure-PyTorch restatement of the AERIS Swin-TrigFlow math: the correctness oracle for every CUDA kernel and the CPU
execution path. Each function cites the reference lines it restates; none of it is used on the GPU hot path.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def get_swin_flop_count(img_dim, B, l, c, d, d_ffnn, p, window_size) -> float:
    """Training FLOPs of one optimizer step (the reference's TFLOPS metric; src/aeris/models/parallel_swin.py:28-53):
    ``6 * [(4 Bw Lw d^2 + 2 Bw Lw^2 d + 3 Bw Lw d_ff d) * l + 2 Bw p c d]``."""
    img_h, img_w = img_dim
    p_dim = p[0] * p[1]
    L_w = window_size[0] * window_size[1]
    assert img_h % (window_size[0] * p[0]) == 0 and img_w % (window_size[1] * p[1]) == 0
    N_w = img_h * img_w / L_w / p_dim
    Bw = B * N_w
    pre_post = 2 * Bw * p_dim * c * d
    qkvo = 4 * Bw * L_w * d ** 2
    fa = 2 * Bw * L_w ** 2 * d
    glu = 3 * Bw * L_w * d_ffnn * d
    return 6 * ((qkvo + fa + glu) * l + pre_post)


def modulate(x: torch.Tensor, shift: torch.Tensor, scale: torch.Tensor | None) -> torch.Tensor:
    """``x * (1 + scale) + shift`` broadcast over tokens (parallel_swin.py:55-59). x: [B, T, D]; shift/scale: [B, D]."""
    if scale is None:
        return x + shift.unsqueeze(1)
    return x * (1 + scale.unsqueeze(1)) + shift.unsqueeze(1)


def timestep_embedding(t: torch.Tensor, dim: int, max_period: float = 10_000) -> torch.Tensor:
    """Sinusoidal embedding, [sin | cos] halves (cos|sin computed, then flipped; parallel_swin.py:61-77). t: [B]."""
    half = dim // 2
    freqs = torch.exp(-math.log(max_period) * torch.arange(0, half, dtype=t.dtype, device=t.device) / half)
    args = t[:, None] * freqs[None]
    emb = torch.cat([torch.cos(args), torch.sin(args)], dim=-1)
    if dim % 2:
        emb = torch.cat([emb, torch.zeros_like(emb[:, :1])], dim=-1)
    return emb.reshape(emb.shape[0], 2, -1).flip(1).reshape(*emb.shape)


def positional_tables(channels: int, h: int, w: int, max_positions: float = 10_000,
                      device=None) -> tuple[torch.Tensor, torch.Tensor]:
    """The two separable factors of :func:`positional_encoding_2d`: a per-row table ``[h, ch]`` for channels
    ``[0, ch)`` and a per-column table ``[w, ch]`` for channels ``[ch, 2 ch)``, ``ch = 2 ceil(channels / 4)``."""
    ch = int(math.ceil(channels / 4) * 2)
    inv_freq = 1.0 / (max_positions ** (torch.arange(0, ch, 2, dtype=torch.float32, device=device) / ch))

    def emb(n):
        s = torch.arange(n, dtype=torch.float32, device=device).unsqueeze(1) * inv_freq
        return torch.stack((s.sin(), s.cos()), dim=-1).flatten(-2, -1)

    return emb(h), emb(w)


def positional_encoding_2d(channels: int, h: int, w: int, max_positions: float = 10_000,
                           dtype=torch.float32, device=None) -> torch.Tensor:
    """Additive 2-D sinusoidal encoding on the input channels, returned as ``[h, w, channels]``
    (parallel_swin.py:120-155: interleaved sin/cos per axis, first half of the channels for rows, second for
    columns, truncated to ``channels``)."""
    ty, tx = positional_tables(channels, h, w, max_positions, device)
    ch = ty.shape[1]
    ey = ty.unsqueeze(1).expand(h, w, ch)
    ex = tx.unsqueeze(0).expand(h, w, ch)
    return torch.cat([ey, ex], dim=-1)[..., :channels].to(dtype)


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()).to(x.dtype)


def rope_2d_cache(ws_y: int, ws_x: int, head_dim: int, base: float = 10_000.0, device=None):
    """(cos, sin), each ``[ws_y * ws_x, head_dim / 2]``, of the axial 2-D rotary embedding of
    parallel_swin.py:158-218: with ``rope_dim = head_dim / 2`` frequencies ``theta_j = base^(-2j / rope_dim)``, the first
    half of a head's (even, odd) channel pairs rotates by ``x * theta``, the second half by ``y * theta`` (x, y: column
    and row of the token inside its window)."""
    rope_dim = head_dim // 2
    theta = 1.0 / (base ** (torch.arange(0, rope_dim, 2, device=device)[: rope_dim // 2].float() / rope_dim))
    idx = torch.arange(ws_y * ws_x, dtype=torch.float32, device=device)
    ang = torch.cat([torch.outer(idx % ws_x, theta), torch.outer(torch.div(idx, ws_x, rounding_mode="floor"), theta)], -1)
    return ang.cos(), ang.sin()


def apply_rope_2d(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, inverse: bool = False) -> torch.Tensor:
    """Rotates the (2i, 2i+1) channel pairs of ``x [..., L, d]`` by the cached angles (``inverse``: by their negatives,
    which is also the transpose of the rotation, i.e. what its backward pass applies to the gradient)."""
    xf = x.float().reshape(*x.shape[:-1], -1, 2)
    s = -sin if inverse else sin
    out = torch.stack([xf[..., 0] * cos - xf[..., 1] * s, xf[..., 1] * cos + xf[..., 0] * s], dim=-1)
    return out.flatten(-2).to(x.dtype)


def window_attention(qkv: torch.Tensor, n_win: int, L: int, heads: int, head_dim: int, rope=None) -> torch.Tensor:
    """softmax(q k^T / sqrt(d)) v per window and head, no mask (parallel_swin.py:257-258). qkv: [n_win*L, 3*h*d]
    with columns ordered (q|k|v, head, d) as produced by ``to_qkv`` (model.py:300). ``rope = (cos, sin)`` applies the
    2-D rotary embedding to q and k first (the reference computes it and then attends on the un-rotated tensors,
    parallel_swin.py:292-294, so parity with it needs ``rope=None``)."""
    q, k, v = qkv.view(n_win, L, 3, heads, head_dim).permute(2, 0, 3, 1, 4)
    if rope is not None:
        q, k = apply_rope_2d(q, *rope), apply_rope_2d(k, *rope)
    o = F.scaled_dot_product_attention(q, k, v, is_causal=False)
    return o.permute(0, 2, 1, 3).reshape(n_win * L, heads * head_dim)


def swiglu(u: torch.Tensor) -> torch.Tensor:
    gate, up = u.chunk(2, dim=-1)
    return F.silu(gate) * up


def block_forward(x: torch.Tensor, mod: torch.Tensor, p: dict, *, n_win_per_sample: int, L: int, heads: int,
                  head_dim: int, after_mod_norm: bool, eps: float, attention=None, mlp=None) -> torch.Tensor:
    """One transformer block on a window-major token stream (parallel_swin.py:454-472).

    x: [B * n_win_per_sample * L, D]; mod: [B, 6 D] = (shift_msa, scale_msa, gate_msa, shift_mlp, scale_mlp,
    gate_mlp); p: weights ``n1, to_qkv, wo, n2, w1, w2``. ``L`` is the number of tokens of a window held locally
    (the whole window unless sequence parallel); ``attention`` overrides the attention call (Ulysses SP), ``mlp`` the
    feed-forward call on the normalised rows (tensor-parallel MLP).
    """
    B = mod.shape[0]
    T, D = x.shape
    xs = x.view(B, T // B, D)
    sh1, sc1, g1, sh2, sc2, g2 = [m.to(x.dtype) for m in mod.chunk(6, dim=1)]

    def pre(xv, shift, scale, w):
        if after_mod_norm:
            return rms_norm(modulate(xv, shift, scale), w, eps)
        return modulate(rms_norm(xv, w, eps), shift, scale)

    h = pre(xs, sh1, sc1, p["n1"]).reshape(T, D)
    qkv = F.linear(h, p["to_qkv"])
    o = (attention or window_attention)(qkv, B * n_win_per_sample, L, heads, head_dim)
    a = F.linear(o, p["wo"]).view(B, T // B, D)
    xs = xs + g1.unsqueeze(1) * a
    h2 = pre(xs, sh2, sc2, p["n2"]).reshape(T, D)
    m = (mlp(h2) if mlp is not None else F.linear(swiglu(F.linear(h2, p["w1"])), p["w2"])).view(B, T // B, D)
    xs = xs + g2.unsqueeze(1) * m
    return xs.reshape(T, D)
