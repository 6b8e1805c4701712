"""Ulysses sequence parallelism: all-to-all that trades a sequence shard of all heads for all of the sequence of a
head shard, as an autograd function whose backward is the inverse exchange.

Reference: ``_SeqAllToAll`` / ``single_all_to_all`` (src/aeris/parallelism/sequence_parallel.py:40-142) used three times
(q, k, v) before and once after attention (src/aeris/models/parallel_swin.py:275-301). Here q, k and v travel in ONE
exchange (the fused qkv tensor is exchanged as a whole), and on backends without ``all_to_all_single`` (gloo, used by
the CPU tests) the exchange is emulated with ``all_gather``.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def _all_to_all_single(out: torch.Tensor, inp: torch.Tensor, group) -> None:
    try:
        backend = dist.get_backend(group)
    except Exception:
        backend = "gloo"
    if backend == "nccl":
        dist.all_to_all_single(out, inp, group=group)
        return
    world = dist.get_world_size(group)
    me = dist.get_rank(group)
    gathered = [torch.empty_like(inp) for _ in range(world)]
    dist.all_gather(gathered, inp.contiguous(), group=group)
    n = inp.shape[0] // world
    for r in range(world):
        out[r * n:(r + 1) * n] = gathered[r][me * n:(me + 1) * n]


def seq_to_head_shard(x: torch.Tensor, group) -> torch.Tensor:
    """x: [W, n_local, Hh, d] (a sequence shard of every head group) -> [W, n_local * SP, Hh / SP, d]
    (the whole sequence of this rank's head groups). ``Hh`` is the head-group axis (3 * heads for a fused qkv)."""
    sp = dist.get_world_size(group)
    W, n, Hh, d = x.shape
    assert Hh % sp == 0
    send = x.reshape(W, n, sp, Hh // sp, d).permute(2, 0, 1, 3, 4).contiguous()     # [sp, W, n, Hh/sp, d]
    recv = torch.empty_like(send)
    _all_to_all_single(recv, send, group)
    return recv.permute(1, 0, 2, 3, 4).reshape(W, sp * n, Hh // sp, d)            # sequence ordered by source rank


def head_to_seq_shard(x: torch.Tensor, group) -> torch.Tensor:
    """Inverse of :func:`seq_to_head_shard`: [W, N, Hh / SP, d] -> [W, N / SP, Hh, d]."""
    sp = dist.get_world_size(group)
    W, N, hl, d = x.shape
    assert N % sp == 0
    send = x.reshape(W, sp, N // sp, hl, d).permute(1, 0, 2, 3, 4).contiguous()      # [sp, W, n, hl, d]
    recv = torch.empty_like(send)
    _all_to_all_single(recv, send, group)
    return recv.permute(1, 2, 0, 3, 4).reshape(W, N // sp, sp * hl, d)


class SeqAllToAll(torch.autograd.Function):
    """``direction='gather_seq'``: sequence shard -> head shard; ``'scatter_seq'``: the inverse. Backward runs the
    opposite exchange (sequence_parallel.py:137-142)."""

    @staticmethod
    def forward(ctx, x, group, direction):
        ctx.group, ctx.direction = group, direction
        return seq_to_head_shard(x, group) if direction == "gather_seq" else head_to_seq_shard(x, group)

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        out = head_to_seq_shard(g, ctx.group) if ctx.direction == "gather_seq" else seq_to_head_shard(g, ctx.group)
        return out, None, None


def sp_window_attention(qkv: torch.Tensor, n_win: int, n_local: int, heads: int, head_dim: int, group,
                        attn_fn) -> torch.Tensor:
    """Window attention over a sequence-sharded stream. qkv: [n_win * n_local, 3 * heads * head_dim] with columns
    (q|k|v, head, d). ``attn_fn(qkv_full [n_win*N, 3*h_local*d], n_win, N, h_local, d) -> [n_win*N, h_local*d]``.
    Token order inside a window after the gather is (source SP rank, local position), the same on q, k and v, and
    attention without positional terms is invariant to it (the reference's RoPE output is discarded,
    parallel_swin.py:292-294)."""
    sp = dist.get_world_size(group)
    assert heads % sp == 0, "heads must divide evenly over the SP ranks"
    hl = heads // sp
    x = qkv.view(n_win, n_local, 3, heads, head_dim)
    # make the head-group axis (qkv, head) split by head first so each rank receives q, k and v of ITS heads
    x = x.permute(0, 1, 3, 2, 4).reshape(n_win, n_local, heads * 3, head_dim)
    full = SeqAllToAll.apply(x, group, "gather_seq")                                # [W, N, 3*hl, d], (head, qkv)
    N = n_local * sp
    full = full.view(n_win, N, hl, 3, head_dim).permute(0, 1, 3, 2, 4).reshape(n_win * N, 3 * hl * head_dim)
    o = attn_fn(full.contiguous(), n_win, N, hl, head_dim)                          # [W*N, hl*d]
    o = o.view(n_win, N, hl, head_dim)
    back = SeqAllToAll.apply(o, group, "scatter_seq")                               # [W, n_local, heads, d]
    return back.reshape(n_win * n_local, heads * head_dim)
