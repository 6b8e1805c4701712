"""CUDA execution of one Swin-TrigFlow block (forward and hand-derived backward) on the sm_100a kernels.

The block is processed in *chunks of whole windows* of one sample: inside a block every token only interacts with its
own window, so a chunk runs modulate+RMSNorm -> QKV GEMM -> window attention -> (wo GEMM + gated residual) ->
modulate+RMSNorm -> (w1 GEMM + SwiGLU) -> (w2 GEMM + gated residual) with a working set of a few GB no matter how
large the image is. Training keeps only the block input (activation checkpointing, absent from the reference and
mandatory for one million tokens per sample); the backward pass recomputes a chunk's internals and immediately
back-propagates through them, accumulating weight gradients in fp32 directly from the GEMM epilogue.

Math restated from src/aeris/models/parallel_swin.py:453-472 (block), :82-104 (SwiGLU), :261-308 (attention).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..ops import attention as A
from ..ops import elementwise as E
from ..ops import gemm as G


@dataclass
class BlockMeta:
    n_win_per_sample: int      # windows of one sample held by this rank
    L: int                     # tokens per window
    heads: int
    head_dim: int
    mode: int                  # E.MODE_MOD_THEN_NORM or E.MODE_NORM_THEN_MOD
    eps: float
    chunk_windows: int = 64
    sp: "SPExchange | None" = None     # Ulysses sequence parallelism: L is then the LOCAL token count of a window
    rope: tuple | None = None          # (cos, sin) [L, head_dim / 2]: optional 2-D rotary embedding of q and k
    tp: object | None = None           # parallel.tensor.TPExchange: w1 / w2 are this rank's shards of the MLP weights


class Workspace:
    """Named scratch tensors, allocated once at the largest size asked for and reused by every block."""

    def __init__(self):
        self._buf: dict[str, torch.Tensor] = {}

    def get(self, name: str, shape: tuple[int, ...], dtype: torch.dtype, device, zero: bool = False) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= s
        b = self._buf.get(name)
        if b is None or b.numel() < n or b.dtype != dtype or b.device != torch.device(device):
            b = torch.empty(n, dtype=dtype, device=device)
            self._buf[name] = b
        v = b[:n].view(*shape)
        if zero:
            v.zero_()
        return v

    def clear(self):
        self._buf.clear()


_WS = Workspace()


def workspace() -> Workspace:
    return _WS


class SPExchange:
    """Symmetric buffers and rank barrier of one Ulysses sequence-parallel group.

    The exchanges of src/aeris/parallelism/sequence_parallel.py:40-86 (three all-to-alls before and one after every
    attention, and their mirrors in backward) do not exist as separate operations here: the QKV GEMM's epilogue stores
    each head's tile into the buffer of the rank that owns the head, and the attention kernels store their output
    (forward) and dQ/dK/dV (backward) into the buffers of the ranks that own the tokens. What is left of the
    collective is a flag barrier between producer and consumer kernels.
    """

    def __init__(self, group, device, timeout_s: float = 20.0):
        import torch.distributed as dist
        from ..engine.fused_dp import RankBarrier
        self.group, self.device = group, torch.device(device)
        self.sp, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.barrier = RankBarrier(group, self.device, timeout_s)
        self._bufs: dict[str, tuple] = {}

    def buffer(self, name: str, shape: tuple[int, int]) -> tuple[torch.Tensor, list[int]]:
        """Symmetric bf16 buffer of at least ``shape`` (every rank must ask for the same sizes in the same order)."""
        import torch.distributed._symmetric_memory as symm_mem
        n = shape[0] * shape[1]
        ent = self._bufs.get(name)
        if ent is None or ent[0].numel() < n:
            t = symm_mem.empty(n, dtype=torch.bfloat16, device=self.device)
            hdl = symm_mem.rendezvous(t, self.group)
            ent = (t, [int(x) for x in hdl.buffer_ptrs], hdl)
            self._bufs[name] = ent
        return ent[0][:n].view(*shape), ent[1]


def _scatter_heads(a: torch.Tensor, w: torch.Tensor, sp: "SPExchange", peers: list[int], n_local: int, L: int,
                   sec_w: int, b_t: bool = False):
    """``a @ w^T`` (or ``a @ w`` with ``b_t``) whose head tiles go to their owner ranks (GEMM-epilogue Ulysses)."""
    import ctypes
    from ..ops import lib as _l
    M, K = a.shape
    N = w.shape[1] if b_t else w.shape[0]
    arr = (ctypes.c_void_p * len(peers))(*peers)
    rc = _l.lib().aeris_gemm_scatter_heads(_l.ptr(a), _l.ptr(w), M, N, K, a.stride(0), w.stride(0), int(b_t), arr,
                                           sp.sp, sp.rank, n_local, L, sec_w, _l.ptr(_l.status_word()),
                                           _l.stream_ptr())
    _l.check(rc, "aeris_gemm_scatter_heads")


def _rope_qk_(qkv: torch.Tensor, meta: BlockMeta, nw: int, inverse: bool = False) -> None:
    """Rotates the q and k sections of a chunk's fused qkv tensor in place (``rope_qk_kernel``; ``inverse`` turns
    gradients with respect to the rotated q, k into gradients with respect to the projections)."""
    assert meta.sp is None, "the rotary embedding is not combined with sequence parallelism"
    cos, sin = meta.rope
    E.rope_qk_(qkv, cos.float().contiguous(), sin.float().contiguous(), meta.L, meta.heads, meta.head_dim, inverse)


def _chunks(meta: BlockMeta):
    step = min(meta.chunk_windows, meta.n_win_per_sample)
    for w0 in range(0, meta.n_win_per_sample, step):
        yield w0, min(step, meta.n_win_per_sample - w0)


def _sp_attention_fwd(meta: BlockMeta, h: torch.Tensor, wqkv: torch.Tensor, nw: int, keep_local: bool):
    """Sequence-parallel attention of one chunk. ``h`` [nw * n_local, D] -> o [nw * n_local, heads * d] (tokens of this
    rank, all heads). Returns (o, state for the backward pass)."""
    import ctypes
    from ..ops import lib as _l
    sp = meta.sp
    n_local, L = meta.L, meta.L * sp.sp
    hl, d = meta.heads // sp.sp, meta.head_dim
    HD = meta.heads * d
    n, nf = nw * n_local, nw * L
    qkv_full, qkv_peers = sp.buffer("qkv_full", (nf, 3 * hl * d))
    o_loc, o_peers = sp.buffer("o_loc", (n, HD))
    _scatter_heads(h, wqkv, sp, qkv_peers, n_local, L, HD)
    sp.barrier()                                  # every rank's q/k/v tiles for my heads have landed
    o_full = _WS.get("sp_o_full", (nf, hl * d), torch.bfloat16, h.device) if keep_local else None
    lse = _WS.get("sp_lse", (nw, hl, L), torch.float32, h.device)
    arr = (ctypes.c_void_p * sp.sp)(*o_peers)
    rc = _l.lib().aeris_attn_fwd_push(_l.ptr(qkv_full), qkv_full.stride(0), hl, _l.ptr(o_full),
                                      o_full.stride(0) if o_full is not None else 0, _l.ptr(lse), nw, L, d,
                                      _l._c_float(1.0 / d ** 0.5), arr, sp.sp, n_local, HD, sp.rank * hl * d,
                                      _l.ptr(_l.status_word()), _l.stream_ptr())
    _l.check(rc, "aeris_attn_fwd_push")
    sp.barrier()                                  # every rank's output rows for my tokens have landed
    return o_loc, (qkv_full, o_full, lse)


def _sp_attention_bwd(meta: BlockMeta, dx1: torch.Tensor, wog: torch.Tensor, nw: int, state):
    """Backward of :func:`_sp_attention_fwd` up to d(qkv) for this rank's tokens [nw * n_local, 3 * heads * d]."""
    import ctypes
    from ..ops import lib as _l
    sp = meta.sp
    qkv_full, o_full, lse = state
    n_local, L = meta.L, meta.L * sp.sp
    hl, d = meta.heads // sp.sp, meta.head_dim
    HD = meta.heads * d
    n, nf = nw * n_local, nw * L
    do_full, do_peers = sp.buffer("do_full", (nf, hl * d))
    dqkv_loc, dq_peers = sp.buffer("dqkv_loc", (n, 3 * HD))
    _scatter_heads(dx1, wog, sp, do_peers, n_local, L, HD, b_t=True)     # d(o) = (dx1 * g1) @ wo, pushed by head
    sp.barrier()
    delta = _WS.get("sp_delta", (nw, hl, L), torch.float32, dx1.device)
    arr = (ctypes.c_void_p * sp.sp)(*dq_peers)
    rc = _l.lib().aeris_attn_bwd_push(_l.ptr(qkv_full), qkv_full.stride(0), hl, _l.ptr(o_full), _l.ptr(do_full),
                                      o_full.stride(0), _l.ptr(lse), _l.ptr(delta), nw, L, d,
                                      _l._c_float(1.0 / d ** 0.5), arr, sp.sp, n_local, 3 * HD, HD, sp.rank * hl * d,
                                      _l.ptr(_l.status_word()), _l.stream_ptr())
    _l.check(rc, "aeris_attn_bwd_push", kernels=2)
    sp.barrier()
    return dqkv_loc


def _tp_mlp_fwd(tp, x1, sc2, sh2, wn2, meta: BlockMeta, w1, w2, g2, act, y_out):
    """Tensor-parallel MLP half of a chunk: ``y = x1 + g2 * reduce_scatter(swiglu(all_gather(h2) @ w1_r^T) @ w2_r^T)``
    with both collectives inside the GEMM kernels (parallel/tensor.py). The modulate+norm kernel writes this rank's
    rows of h2 straight into the all-gather buffer; the barrier inside the reduce-scatter orders a chunk's reads
    before the next chunk's pushes."""
    from ..parallel import tensor as TP
    n, D = x1.shape
    M = tp.tp * n
    a_buf, peers = tp.buffer("ag_x", (M, D))
    E.modnorm_fwd(x1, sc2, sh2, wn2, mode=meta.mode, eps=meta.eps, out=a_buf[tp.rank * n:(tp.rank + 1) * n])
    tp.barrier()
    TP.gemm_allgather_a(tp, a_buf, peers, w1, out=act[:M], epi=G.EPI_SWIGLU)
    TP.gemm_reduce_scatter(tp, act[:M], w2, resid=x1, gate=g2, out=y_out)


def block_forward(x: torch.Tensor, mod: torch.Tensor, meta: BlockMeta, wn1, wqkv, wo, wn2, w1, w2,
                  out: torch.Tensor | None = None, gather=None) -> torch.Tensor:
    """x: [B * n_win * L, D] bf16 window-major; mod: [B, 6D] fp32 (shift1, scale1, gate1, shift2, scale2, gate2).

    ``gather = (table, peer_ptrs, src)``: ``x`` is then an EMPTY buffer in this block's window layout; the first
    modulate+norm kernel of every chunk pulls its rows through the table from ``src`` on this or a peer GPU (the
    re-partition / halo exchange of a shifted layer) and writes them into ``x`` on the way."""
    T, D = x.shape
    B = mod.shape[0]
    F = w2.shape[1]
    HD = meta.heads * meta.head_dim
    rows_per_sample = meta.n_win_per_sample * meta.L
    assert T == B * rows_per_sample
    y = out if out is not None else torch.empty_like(x)
    ws, dev, bf = _WS, x.device, torch.bfloat16
    cmax = min(meta.chunk_windows, meta.n_win_per_sample) * meta.L
    h = ws.get("h", (cmax, D), bf, dev)
    qkv = ws.get("qkv", (cmax, 3 * HD), bf, dev)
    o = ws.get("o", (cmax, HD), bf, dev)
    x1 = ws.get("x1", (cmax, D), bf, dev)
    tpn = meta.tp.tp if meta.tp is not None else 1       # gathered rows x local features: the same element count
    act = ws.get("act", (cmax * tpn, F), bf, dev)
    lse = ws.get("lse", (cmax * meta.heads,), torch.float32, dev)
    mod = mod.contiguous()
    for b in range(B):
        sh1, sc1, g1, sh2, sc2, g2 = [mod[b, i * D:(i + 1) * D] for i in range(6)]
        for w0, nw in _chunks(meta):
            r0 = b * rows_per_sample + w0 * meta.L
            n = nw * meta.L
            xc = x[r0:r0 + n]
            if gather is not None:
                table, peers, src = gather
                E.modnorm_fwd(None, sc1, sh1, wn1, mode=meta.mode, eps=meta.eps, out=h[:n],
                              gather_idx=table[r0:r0 + n], peer_ptrs=peers, x_out=xc, rows=n,
                              src_rows=src.shape[0])
            else:
                E.modnorm_fwd(xc, sc1, sh1, wn1, mode=meta.mode, eps=meta.eps, out=h[:n])
            if meta.sp is None:
                G.gemm(h[:n], wqkv, out=qkv[:n])
                if meta.rope is not None:
                    _rope_qk_(qkv[:n], meta, nw)
                A.attn_fwd(qkv[:n], nw, meta.L, meta.heads, meta.head_dim, out=o[:n],
                           lse=lse[:n * meta.heads].view(nw, meta.heads, meta.L))
                oc = o[:n]
            else:
                oc = _sp_attention_fwd(meta, h[:n], wqkv, nw, keep_local=False)[0]
            G.gemm(oc, wo, out=x1[:n], epi=G.EPI_GATE_RESID, resid=xc, gate=g1)
            if meta.tp is not None:
                _tp_mlp_fwd(meta.tp, x1[:n], sc2, sh2, wn2, meta, w1, w2, g2, act, y[r0:r0 + n])
                continue
            E.modnorm_fwd(x1[:n], sc2, sh2, wn2, mode=meta.mode, eps=meta.eps, out=h[:n])
            G.gemm(h[:n], w1, out=act[:n], epi=G.EPI_SWIGLU)
            G.gemm(act[:n], w2, out=y[r0:r0 + n], epi=G.EPI_GATE_RESID, resid=x1[:n], gate=g2)
    return y


def block_backward(x: torch.Tensor, mod: torch.Tensor, dy: torch.Tensor, meta: BlockMeta, wn1, wqkv, wo, wn2, w1, w2,
                   grads: dict[str, torch.Tensor], dx: torch.Tensor | None = None):
    """Recompute-and-backpropagate. ``grads`` maps n1, to_qkv, wo, n2, w1, w2 to fp32 accumulators (+=).
    Returns (dx bf16, dmod [B, 6D] fp32). ``dx`` may alias ``dy``."""
    T, D = x.shape
    B = mod.shape[0]
    F = w2.shape[1]
    HD = meta.heads * meta.head_dim
    rows_per_sample = meta.n_win_per_sample * meta.L
    ws, dev, bf, f32 = _WS, x.device, torch.bfloat16, torch.float32
    cmax = min(meta.chunk_windows, meta.n_win_per_sample) * meta.L
    h1 = ws.get("h", (cmax, D), bf, dev)
    qkv = ws.get("qkv", (cmax, 3 * HD), bf, dev)
    o = ws.get("o", (cmax, HD), bf, dev)
    x1 = ws.get("x1", (cmax, D), bf, dev)
    tp = meta.tp
    tpn = tp.tp if tp is not None else 1
    act = ws.get("act", (cmax * tpn, F), bf, dev)
    lse = ws.get("lse", (cmax * meta.heads,), f32, dev)
    h2 = ws.get("h2", (cmax, D), bf, dev)
    u = ws.get("u", (cmax * tpn, 2 * F), bf, dev)
    dh = ws.get("dh", (cmax, D), bf, dev)
    dx1 = ws.get("dx1", (cmax, D), bf, dev)
    d_o = ws.get("d_o", (cmax, HD), bf, dev)
    dqkv = ws.get("dqkv", (cmax, 3 * HD), bf, dev)
    delta = ws.get("delta", (cmax * meta.heads,), f32, dev)
    w2g = ws.get("w2g", tuple(w2.shape), bf, dev)
    wog = ws.get("wog", tuple(wo.shape), bf, dev)
    G2 = ws.get("G2", tuple(w2.shape), f32, dev, zero=True)   # dy^T act  (ungated w2 gradient of one sample)
    Go = ws.get("Go", tuple(wo.shape), f32, dev, zero=True)   # dx1^T o
    dmod = torch.zeros((B, 6 * D), dtype=f32, device=dev)
    if dx is None:
        dx = torch.empty_like(x)
    mod = mod.contiguous()
    ksplit_tok = 4
    for b in range(B):
        sh1, sc1, g1, sh2, sc2, g2 = [mod[b, i * D:(i + 1) * D] for i in range(6)]
        dsh1, dsc1, dg1, dsh2, dsc2, dg2 = [dmod[b, i * D:(i + 1) * D] for i in range(6)]
        E.scale_rows(w2, g2, out=w2g)
        E.scale_rows(wo, g1, out=wog)
        for w0, nw in _chunks(meta):
            r0 = b * rows_per_sample + w0 * meta.L
            n = nw * meta.L
            xc, dyc = x[r0:r0 + n], dy[r0:r0 + n]
            lse_c = lse[:n * meta.heads].view(nw, meta.heads, meta.L)
            # ---- recompute the chunk's forward internals
            E.modnorm_fwd(xc, sc1, sh1, wn1, mode=meta.mode, eps=meta.eps, out=h1[:n])
            if meta.sp is None:
                G.gemm(h1[:n], wqkv, out=qkv[:n])
                if meta.rope is not None:
                    _rope_qk_(qkv[:n], meta, nw)
                A.attn_fwd(qkv[:n], nw, meta.L, meta.heads, meta.head_dim, out=o[:n], lse=lse_c)
                oc = o[:n]
            else:
                oc, sp_state = _sp_attention_fwd(meta, h1[:n], wqkv, nw, keep_local=True)
            G.gemm(oc, wo, out=x1[:n], epi=G.EPI_GATE_RESID, resid=xc, gate=g1)
            if tp is not None:
                # tensor-parallel MLP half: h2 and dy are gathered over the group inside the two GEMMs that consume
                # them, the partial dh2 is reduced and scattered by the epilogue of the GEMM that produces it
                from ..parallel import tensor as TP
                Mg = tpn * n
                sl = slice(tp.rank * n, (tp.rank + 1) * n)
                x_buf, x_peers = tp.buffer("ag_x", (Mg, D))
                g_buf, g_peers = tp.buffer("ag_dy", (Mg, D))
                E.modnorm_fwd(x1[:n], sc2, sh2, wn2, mode=meta.mode, eps=meta.eps, out=x_buf[sl])
                g_buf[sl].copy_(dyc)
                tp.barrier()
                TP.gemm_allgather_a(tp, x_buf, x_peers, w1, out=act[:Mg], epi=G.EPI_SWIGLU_BOTH, aux=u[:Mg])
                TP.gemm_allgather_a(tp, g_buf, g_peers, w2g, b_t=True, out=u[:Mg], epi=G.EPI_SWIGLU_BWD, resid=u[:Mg])
                G.gemm(g_buf, act[:Mg], a_t=True, b_t=True, out=G2, epi=G.EPI_ACC_F32, k_splits=ksplit_tok)
                G.gemm(u[:Mg], x_buf, a_t=True, b_t=True, out=grads["w1"], epi=G.EPI_ACC_F32, k_splits=ksplit_tok)
                TP.gemm_reduce_scatter(tp, u[:Mg], w1, b_t=True, name="rs_dx", out=dh[:n])
            else:
                E.modnorm_fwd(x1[:n], sc2, sh2, wn2, mode=meta.mode, eps=meta.eps, out=h2[:n])
                G.gemm(h2[:n], w1, out=act[:n], epi=G.EPI_SWIGLU_BOTH, aux=u[:n])     # act and the raw [gate | up]
                # ---- MLP half: y = x1 + g2 * (act @ w2^T)
                G.gemm(dyc, act[:n], a_t=True, b_t=True, out=G2, epi=G.EPI_ACC_F32, k_splits=ksplit_tok)
                # dact = (dy * g2) @ w2 never reaches memory: the epilogue turns it into du, overwriting u
                G.gemm(dyc, w2g, b_t=True, out=u[:n], epi=G.EPI_SWIGLU_BWD, resid=u[:n])
                G.gemm(u[:n], w1, b_t=True, out=dh[:n])                                # dh2 = du @ w1
                G.gemm(u[:n], h2[:n], a_t=True, b_t=True, out=grads["w1"], epi=G.EPI_ACC_F32, k_splits=ksplit_tok)
            E.modnorm_bwd(x1[:n], dh[:n], dyc, sc2, sh2, wn2, mode=meta.mode, eps=meta.eps, dx=dx1[:n],
                          dscale=dsc2, dshift=dsh2, dw=grads["n2"])
            # ---- attention half: x1 = x + g1 * (o @ wo^T)
            G.gemm(dx1[:n], oc, a_t=True, b_t=True, out=Go, epi=G.EPI_ACC_F32, k_splits=ksplit_tok)
            if meta.sp is None:
                G.gemm(dx1[:n], wog, b_t=True, out=d_o[:n])                            # do = (dx1 * g1) @ wo
                A.attn_bwd(qkv[:n], o[:n], d_o[:n], lse_c, nw, meta.L, meta.heads, meta.head_dim, dqkv=dqkv[:n],
                           delta=delta[:n * meta.heads].view(nw, meta.heads, meta.L))
                if meta.rope is not None:
                    _rope_qk_(dqkv[:n], meta, nw, inverse=True)
                dq_c = dqkv[:n]
            else:
                dq_c = _sp_attention_bwd(meta, dx1[:n], wog, nw, sp_state)
            G.gemm(dq_c, wqkv, b_t=True, out=dh[:n])                                   # dh1 = dqkv @ wqkv
            G.gemm(dq_c, h1[:n], a_t=True, b_t=True, out=grads["to_qkv"], epi=G.EPI_ACC_F32, k_splits=ksplit_tok)
            E.modnorm_bwd(xc, dh[:n], dx1[:n], sc1, sh1, wn1, mode=meta.mode, eps=meta.eps, dx=dx[r0:r0 + n],
                          dscale=dsc1, dshift=dsh1, dw=grads["n1"])
        # per-sample gate handling: dW += g * G ; dg = rowsum(W * G) ; G <- 0
        E.gate_grad_finalize(G2, w2, g2, grads["w2"], dg2)
        E.gate_grad_finalize(Go, wo, g1, grads["wo"], dg1)
    return dx, dmod


def _pool_alloc(peer_fn, gradient: bool = False):
    """The peer-readable buffer allocator that belongs to a halo exchange's ``peer_fn`` (or None)."""
    return getattr(getattr(peer_fn, "__self__", None), "gradient_buffer" if gradient else "output_buffer", None)


class FusedBlock(torch.autograd.Function):
    """Autograd wrapper: saves only the block input; weight gradients go to ``param.main_grad`` (fp32) when the
    engine provides one, otherwise they are returned to autograd."""

    @staticmethod
    def forward(ctx, x, mod, meta, wn1, wqkv, wo, wn2, w1, w2, regroup=None, out_alloc=None):
        """``regroup = (table_fwd, table_bwd, peer_fn)`` fuses the preceding window re-partition into this block: the
        incoming stream ``x`` is in the previous layout (published to the WP peers when ``peer_fn`` is given) and the
        first modulate+norm kernel gathers this block's rows from it. ``out_alloc(rows, cols, dtype)``: where to put the
        output when the caller knows that it will be re-partitioned next (a peer-readable buffer: no publish copy)."""
        ctx.meta = meta
        ctx.regroup = regroup
        out = out_alloc(x.shape[0], x.shape[1], x.dtype) if out_alloc is not None else None
        if regroup is not None:
            table_fwd, _, peer_fn = regroup
            peers = peer_fn(x, "fwd") if peer_fn is not None else [x.data_ptr()]
            xg = torch.empty((table_fwd.numel(), x.shape[1]), dtype=x.dtype, device=x.device)
            y = block_forward(xg, mod.float(), meta, wn1, wqkv, wo, wn2, w1, w2, out=out,
                              gather=(table_fwd, peers, x))
            x = xg
        else:
            y = block_forward(x, mod.float(), meta, wn1, wqkv, wo, wn2, w1, w2, out=out)
        ctx.save_for_backward(x, mod, wn1, wqkv, wo, wn2, w1, w2)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, mod, wn1, wqkv, wo, wn2, w1, w2 = ctx.saved_tensors
        params = {"n1": wn1, "to_qkv": wqkv, "wo": wo, "n2": wn2, "w1": w1, "w2": w2}
        grads, ret = {}, {}
        for k, p in params.items():
            mg = getattr(p, "main_grad", None)
            if mg is not None:
                grads[k] = mg.view(p.shape) if mg.dim() != p.dim() else mg
                ret[k] = None
            else:
                grads[k] = torch.zeros(p.shape, dtype=torch.float32, device=p.device)
                ret[k] = grads[k]
        dy = dy.contiguous()
        dx, dmod = block_backward(x, mod.float(), dy, ctx.meta, wn1, wqkv, wo, wn2, w1, w2, grads, dx=dy)
        if ctx.regroup is not None:
            _, table_bwd, peer_fn = ctx.regroup
            peers = peer_fn(dx, "bwd") if peer_fn is not None else [dx.data_ptr()]
            # the gathered gradient is the next (earlier) layer's dy, which that layer turns into its dx in place and
            # publishes in turn: put it into the other peer-readable buffer straight away
            alloc = _pool_alloc(peer_fn, gradient=True)
            back = (alloc(table_bwd.numel(), dx.shape[1], dx.dtype) if alloc is not None else
                    torch.empty((table_bwd.numel(), dx.shape[1]), dtype=dx.dtype, device=dx.device))
            E.gather_rows(table_bwd, peers, back, src_rows=dx.shape[0])
            dx = back
        out = [ret[k].to(params[k].dtype) if ret[k] is not None else None
               for k in ("n1", "to_qkv", "wo", "n2", "w1", "w2")]
        return (dx, dmod.to(mod.dtype), None, *out, None, None)


class GemvLinearFn(torch.autograd.Function):
    """``silu?(x) @ W^T + b`` for the handful of rows of a modulation MLP (one row per sample): the forward streams the
    weight once through the GEMV kernel; weight gradients are rank-B updates added to the fp32 gradient buffers."""

    @staticmethod
    def forward(ctx, x, W, b, silu_in: bool):
        from ..ops import diffusion as DF
        x32 = x.float().contiguous()
        y = DF.gemv_bias_act(W.detach(), b.detach().float() if b is not None else None, x32, act=0, silu_in=silu_in)
        ctx.silu_in, ctx.x_dtype = silu_in, x.dtype
        ctx.save_for_backward(x32, W, b)
        return y

    @staticmethod
    def backward(ctx, dy):
        from .fused_io import _grad_slot
        x32, W, b = ctx.saved_tensors
        dy = dy.float()
        sig = torch.sigmoid(x32) if ctx.silu_in else None
        h = x32 * sig if ctx.silu_in else x32
        sW, rW = _grad_slot(W)
        sW.addmm_(dy.t(), h)
        rb = None
        if b is not None:
            sb, rb = _grad_slot(b)
            sb += dy.sum(0)
        dx = (dy.to(W.dtype) @ W).float()
        if ctx.silu_in:
            dx = dx * (sig * (1 + x32 * (1 - sig)))
        return (dx.to(ctx.x_dtype), rW.to(W.dtype) if rW is not None else None,
                rb.to(b.dtype) if rb is not None else None, None)


def modulation(seq: torch.nn.Sequential, emb: torch.Tensor) -> torch.Tensor:
    """The AdaLN modulation MLP ``[Linear,] SiLU, Linear`` (src/aeris/models/parallel_swin.py:321-325) of at most 8
    samples on the GEMV kernel; fp32 result ``[B, out]``."""
    if emb.shape[0] > 8:
        return seq(emb.to(seq[-1].weight.dtype)).float()
    x = emb
    if len(seq) == 3:
        x = GemvLinearFn.apply(x, seq[0].weight, seq[0].bias, False)
    return GemvLinearFn.apply(x, seq[-1].weight, seq[-1].bias, True)


class Regroup(torch.autograd.Function):
    """Row gather between two window layouts through a table; the backward pass is the gather with the inverse
    table. ``peers`` lists the base addresses of every WP rank's source buffer (just the local one without WP)."""

    @staticmethod
    def forward(ctx, x, table_fwd, table_bwd, peer_fn):
        ctx.table_bwd, ctx.peer_fn = table_bwd, peer_fn
        out = torch.empty((table_fwd.numel(), x.shape[1]), dtype=x.dtype, device=x.device)
        peers = peer_fn(x, "fwd") if peer_fn is not None else [x.data_ptr()]
        E.gather_rows(table_fwd, peers, out, src_rows=x.shape[0])
        return out

    @staticmethod
    def backward(ctx, dy):
        dy = dy.contiguous()
        peers = ctx.peer_fn(dy, "bwd") if ctx.peer_fn is not None else [dy.data_ptr()]
        alloc = _pool_alloc(ctx.peer_fn, gradient=True)      # the previous layer's dy: see FusedBlock.backward
        out = (alloc(ctx.table_bwd.numel(), dy.shape[1], dy.dtype) if alloc is not None else
               torch.empty((ctx.table_bwd.numel(), dy.shape[1]), dtype=dy.dtype, device=dy.device))
        E.gather_rows(ctx.table_bwd, peers, out, src_rows=dy.shape[0])
        return out, None, None, None
