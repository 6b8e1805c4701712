"""Tensor-parallel SwiGLU MLP over the GPUs of one NVSwitch node, with both collectives fused into the GEMMs.

The token rows are sharded over the ``tp`` ranks (the layout Ulysses sequence parallelism already gives the residual
stream), ``w1`` is split by output features and ``w2`` by input features:

    X_full = all_gather_rows(h)                 -- fused: a copier thread of the w1 GEMM pushes this rank's rows to the peers (bulk copies)
    U_r    = X_full @ w1_r^T ; act_r = silu(gate) * up          while its tiles start on the local rows
    Y      = reduce_scatter_rows(act_r @ w2_r^T)  -- fused: the w2 GEMM's epilogue stores each bf16 partial tile into
                                                    the owner rank's slot buffer; the owner sums its slots

The reference has no tensor parallelism (its MLP, src/aeris/models/parallel_swin.py:82-104, is replicated over the
sequence-parallel ranks); this halves / quarters the MLP weights, gradients and optimizer state per GPU for the
larger model sizes. The backward pass uses the same two kernels: all-gather of dY fused into the d(act) product,
reduce-scatter of the partial dX fused into the d(h) product.

CPU / gloo: :func:`tp_mlp_reference` states the same math with ``torch.distributed`` collectives.
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from ..ops import gemm as G
from ..ops import lib as _l


class TPExchange:
    """Symmetric buffers, arrival counters and the rank barrier of one tensor-parallel group."""

    def __init__(self, group, device, timeout_s: float = 20.0):
        from ..engine.fused_dp import RankBarrier
        self.group, self.device = group, torch.device(device)
        self.tp, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.barrier = RankBarrier(group, self.device, timeout_s)
        import torch.distributed._symmetric_memory as symm_mem
        # arrival words of the fused all-gather: word s of rank r counts the CTAs of rank s that have pushed their
        # slice into r's buffer; they only ever grow (expected value = calls so far x CTAs per call)
        self.counters = symm_mem.empty(8, dtype=torch.int32, device=self.device)
        self.counters.zero_()
        self._cnt_hdl = symm_mem.rendezvous(self.counters, group)
        self.counter_ptrs = (ctypes.c_void_p * self.tp)(*[int(x) for x in self._cnt_hdl.buffer_ptrs])
        self.ag_calls = 0
        self._bufs: dict[str, tuple] = {}
        dist.barrier(group)

    def buffer(self, name: str, shape: tuple[int, int]):
        """Symmetric bf16 buffer (every rank asks for the same names and sizes in the same order)."""
        import torch.distributed._symmetric_memory as symm_mem
        n = shape[0] * shape[1]
        ent = self._bufs.get(name)
        if ent is None or ent[0].numel() < n:
            t = symm_mem.empty(n, dtype=torch.bfloat16, device=self.device)
            hdl = symm_mem.rendezvous(t, self.group)
            ent = (t, (ctypes.c_void_p * self.tp)(*[int(x) for x in hdl.buffer_ptrs]), hdl)
            self._bufs[name] = ent
        return ent[0][:n].view(*shape), ent[1]


def gemm_allgather_a(tpx: TPExchange, a_buf: torch.Tensor, peers, b: torch.Tensor, *, out: torch.Tensor,
                     b_t: bool = False, epi: int = G.EPI_STORE, resid: torch.Tensor | None = None,
                     aux: torch.Tensor | None = None) -> torch.Tensor:
    """``out = epi(all_gather_rows(a) @ b^T)``: ``a_buf`` is the [tp * n_loc, K] symmetric buffer whose chunk ``rank``
    holds this rank's rows; afterwards it holds every rank's rows."""
    M, K = a_buf.shape
    N = b.shape[1] if b_t else b.shape[0]
    swiglu_f = 0
    if epi in (G.EPI_SWIGLU, G.EPI_SWIGLU_BOTH):
        swiglu_f = N // 2
    elif epi == G.EPI_SWIGLU_BWD:
        swiglu_f = N
    tpx.ag_calls += 1
    rc = _l.lib().aeris_gemm_allgather_a(
        _l.ptr(a_buf), peers, tpx.counter_ptrs, tpx.tp, tpx.rank, M // tpx.tp, ctypes.c_uint(tpx.ag_calls),
        _l.ptr(b), _l.ptr(out), N, K, b.stride(0), out.stride(0), int(b_t), epi, _l.ptr(resid),
        resid.stride(0) if resid is not None else 0, _l.ptr(aux), aux.stride(0) if aux is not None else 0, swiglu_f,
        _l.ptr(_l.status_word()), _l.stream_ptr())
    _l.check(rc, "aeris_gemm_allgather_a")
    return out


def gemm_reduce_scatter(tpx: TPExchange, a: torch.Tensor, b: torch.Tensor, *, b_t: bool = False,
                        resid: torch.Tensor | None = None, gate: torch.Tensor | None = None,
                        out: torch.Tensor | None = None, name: str = "rs") -> torch.Tensor:
    """``out[n_loc, N] = resid + gate * sum_ranks (a_r @ b_r^T)[rows of this rank]`` with the scatter fused into the
    GEMM epilogue (bf16 partial tiles pushed to the owner) and the sum done by the owner."""
    M, K = a.shape
    N = b.shape[1] if b_t else b.shape[0]
    n_loc = M // tpx.tp
    slots, peers = tpx.buffer(name, (tpx.tp * n_loc, N))
    rc = _l.lib().aeris_gemm_rs_push(_l.ptr(a), _l.ptr(b), M, N, K, a.stride(0), b.stride(0), int(b_t), peers,
                                     tpx.tp, tpx.rank, n_loc, N, _l.ptr(_l.status_word()), _l.stream_ptr())
    _l.check(rc, "aeris_gemm_rs_push")
    tpx.barrier()
    if out is None:
        out = torch.empty((n_loc, N), dtype=torch.bfloat16, device=a.device)
    rc = _l.lib().aeris_rs_finalize(_l.ptr(slots), tpx.tp, _l._c_ll(n_loc), N, _l.ptr(resid), _l.ptr(gate),
                                    _l.ptr(out), _l.stream_ptr())
    _l.check(rc, "aeris_rs_finalize")
    return out


def _grad_slot(p):
    from ..models.fused_io import _grad_slot as gs
    return gs(p)


class TPMlpFn(torch.autograd.Function):
    """``y = [resid +] [gate *] swiglu(all_gather(h) @ w1_r^T) @ w2_r^T`` reduced and scattered back to row shards.
    ``w1_r``: [2 F / tp, D] (this rank's gate rows, then its up rows), ``w2_r``: [D, F / tp]. Keeps only ``h``."""

    @staticmethod
    def forward(ctx, h, w1, w2, tpx: TPExchange):
        n_loc, D = h.shape
        M = tpx.tp * n_loc
        F2 = w1.shape[0]
        a_buf, peers = tpx.buffer("ag_x", (M, D))
        a_buf[tpx.rank * n_loc:(tpx.rank + 1) * n_loc].copy_(h)
        tpx.barrier()
        act = torch.empty((M, F2 // 2), dtype=torch.bfloat16, device=h.device)
        gemm_allgather_a(tpx, a_buf, peers, w1, out=act, epi=G.EPI_SWIGLU)
        y = gemm_reduce_scatter(tpx, act, w2)
        ctx.tpx = tpx
        ctx.save_for_backward(h, w1, w2)
        return y

    @staticmethod
    def backward(ctx, dy):
        h, w1, w2 = ctx.saved_tensors
        tpx = ctx.tpx
        n_loc, D = h.shape
        M = tpx.tp * n_loc
        F2 = w1.shape[0]
        dev = h.device
        sl = slice(tpx.rank * n_loc, (tpx.rank + 1) * n_loc)
        x_buf, x_peers = tpx.buffer("ag_x", (M, D))
        g_buf, g_peers = tpx.buffer("ag_dy", (M, D))
        x_buf[sl].copy_(h)
        g_buf[sl].copy_(dy)
        tpx.barrier()
        act = torch.empty((M, F2 // 2), dtype=torch.bfloat16, device=dev)
        u = torch.empty((M, F2), dtype=torch.bfloat16, device=dev)
        gemm_allgather_a(tpx, x_buf, x_peers, w1, out=act, epi=G.EPI_SWIGLU_BOTH, aux=u)     # recompute; x gathered
        gemm_allgather_a(tpx, g_buf, g_peers, w2, out=u, b_t=True, epi=G.EPI_SWIGLU_BWD, resid=u)   # du; dy gathered
        s2, r2 = _grad_slot(w2)
        G.gemm(g_buf, act, a_t=True, b_t=True, out=s2, epi=G.EPI_ACC_F32, k_splits=4)         # dW2_r = dY^T act_r
        s1, r1 = _grad_slot(w1)
        G.gemm(u, x_buf, a_t=True, b_t=True, out=s1, epi=G.EPI_ACC_F32, k_splits=4)           # dW1_r = dU_r^T X
        dh = gemm_reduce_scatter(tpx, u, w1, b_t=True, name="rs_dx")                          # dX = RS(dU_r @ w1_r)
        return (dh, r1.to(w1.dtype) if r1 is not None else None, r2.to(w2.dtype) if r2 is not None else None, None)


def shard_mlp_weights(w1: torch.Tensor, w2: torch.Tensor, tp: int, rank: int):
    """Rank ``rank``'s shards of the full ``w1`` [2F, D] (gate rows, then up rows) and ``w2`` [D, F]."""
    F = w2.shape[1]
    f = F // tp
    w1_r = torch.cat([w1[rank * f:(rank + 1) * f], w1[F + rank * f:F + (rank + 1) * f]], dim=0).contiguous()
    w2_r = w2[:, rank * f:(rank + 1) * f].contiguous()
    return w1_r, w2_r


def tp_mlp_reference(h: torch.Tensor, w1_r: torch.Tensor, w2_r: torch.Tensor, group) -> torch.Tensor:
    """The same computation with torch.distributed collectives (any backend; differentiable through autograd's
    functional collectives is not needed here: used for forward parity and on CPU)."""
    tp, rank = dist.get_world_size(group), dist.get_rank(group)
    parts = [torch.empty_like(h) for _ in range(tp)]
    dist.all_gather(parts, h.contiguous(), group=group)
    x = torch.cat(parts)
    u = x @ w1_r.t()
    f = u.shape[1] // 2
    act = torch.nn.functional.silu(u[:, :f]) * u[:, f:]
    y = (act @ w2_r.t()).float()
    dist.all_reduce(y, group=group)
    n_loc = h.shape[0]
    return y[rank * n_loc:(rank + 1) * n_loc].to(h.dtype)


class TPMlpCollective(torch.autograd.Function):
    """The tensor-parallel SwiGLU MLP with ``torch.distributed`` collectives and a hand-written backward pass (any
    backend; the CPU / gloo path of the model and the statement of what the fused kernels compute):
    ``y = reduce_scatter_rows(swiglu(all_gather_rows(h) @ w1_r^T) @ w2_r^T)``."""

    @staticmethod
    def _gather(t, group):
        parts = [torch.empty_like(t) for _ in range(dist.get_world_size(group))]
        dist.all_gather(parts, t.contiguous(), group=group)
        return torch.cat(parts)

    @staticmethod
    def _scatter_sum(t, group):
        t = t.float().contiguous()
        dist.all_reduce(t, group=group)
        n = t.shape[0] // dist.get_world_size(group)
        r = dist.get_rank(group)
        return t[r * n:(r + 1) * n]

    @staticmethod
    def forward(ctx, h, w1, w2, group):
        x = TPMlpCollective._gather(h, group)
        u = x @ w1.t()
        f = u.shape[1] // 2
        act = torch.nn.functional.silu(u[:, :f]) * u[:, f:]
        ctx.group = group
        ctx.save_for_backward(h, w1, w2)
        return TPMlpCollective._scatter_sum(act @ w2.t(), group).to(h.dtype)

    @staticmethod
    def backward(ctx, dy):
        h, w1, w2 = ctx.saved_tensors
        x = TPMlpCollective._gather(h, ctx.group)
        g = TPMlpCollective._gather(dy, ctx.group)
        u = x @ w1.t()
        f = u.shape[1] // 2
        gate, up = u[:, :f].float(), u[:, f:].float()
        sig = torch.sigmoid(gate)
        act = (gate * sig * up).to(h.dtype)
        dact = (g @ w2).float()
        du = torch.cat([dact * up * sig * (1 + gate * (1 - sig)), dact * gate * sig], dim=1).to(h.dtype)
        dw2 = g.t() @ act
        dw1 = du.t() @ x
        dh = TPMlpCollective._scatter_sum(du @ w1, ctx.group).to(h.dtype)
        return dh, dw1, dw2, None


def tp_kind(name: str, p=None) -> str | None:
    """"w1" / "w2" for the tensor-parallel-sharded weights of a model built with ``tp > 1``, else None."""
    k = getattr(p, "tp_shard", None)
    if k is not None:
        return k
    if "latent_embed" in name:           # the noise-level embedding's own w1 / w2 are replicated
        return None
    if name.endswith(".w1.weight"):
        return "w1"
    if name.endswith(".w2.weight"):
        return "w2"
    return None


def shard_tensor(kind: str, full: torch.Tensor, tp: int, rank: int) -> torch.Tensor:
    """Rank ``rank``'s shard of a full ``w1``-shaped [2F, D] or ``w2``-shaped [D, F] tensor (weights, masters, Adam
    moments and EMA all share the parameter's shape)."""
    if kind == "w1":
        F = full.shape[0] // 2
        f = F // tp
        return torch.cat([full[rank * f:(rank + 1) * f], full[F + rank * f:F + (rank + 1) * f]], dim=0).contiguous()
    f = full.shape[1] // tp
    return full[:, rank * f:(rank + 1) * f].contiguous()


def unshard_tensors(kind: str, shards: list[torch.Tensor]) -> torch.Tensor:
    """Inverse of :func:`shard_tensor` over the shards of all ranks, in rank order."""
    if kind == "w1":
        f = shards[0].shape[0] // 2
        return torch.cat([s[:f] for s in shards] + [s[f:] for s in shards], dim=0)
    return torch.cat(shards, dim=1)


def gather_full(kind: str, shard: torch.Tensor, group) -> torch.Tensor:
    """Collective over the tensor-parallel group: the full tensor on every rank (on the shard's device)."""
    parts = [torch.empty_like(shard) for _ in range(dist.get_world_size(group))]
    dist.all_gather(parts, shard.contiguous(), group=group)
    return unshard_tensors(kind, parts)


def full_state_dict(named: dict[str, torch.Tensor], group) -> dict[str, torch.Tensor]:
    """A dict of per-parameter tensors with the tensor-parallel shards replaced by the gathered full tensors
    (collective: every rank of ``group`` calls it with the same keys in the same order)."""
    out = {}
    for k, v in named.items():
        kind = tp_kind(k)
        if kind is None:
            out[k] = v
        else:
            dev = v.device
            if dist.get_backend(group) == "nccl" and not v.is_cuda:
                v = v.cuda()
            out[k] = gather_full(kind, v, group).to(dev)
    return out


def fit_to_shard(name: str, t: torch.Tensor, like: torch.Tensor, tp: int, rank: int) -> torch.Tensor:
    """``t`` as stored in a checkpoint (full size) cut down to this rank's shard when ``like`` is a shard."""
    kind = tp_kind(name)
    if kind is None or tuple(t.shape) == tuple(like.shape) or tp <= 1:
        return t
    return shard_tensor(kind, t, tp, rank)


class TPFeedForward(torch.nn.Module):
    """SwiGLU feed-forward whose weights are sharded over a tensor-parallel group (see module docstring)."""

    def __init__(self, dim: int, hidden: int, tp: int, dtype=torch.bfloat16):
        super().__init__()
        assert hidden % tp == 0
        self.w1 = torch.nn.Parameter(torch.empty(2 * hidden // tp, dim, dtype=dtype))
        self.w2 = torch.nn.Parameter(torch.empty(dim, hidden // tp, dtype=dtype))
        torch.nn.init.normal_(self.w1, std=dim ** -0.5)
        torch.nn.init.normal_(self.w2, std=hidden ** -0.5)
        self.tpx: TPExchange | None = None

    def forward(self, h: torch.Tensor, group=None) -> torch.Tensor:
        if h.is_cuda:
            if self.tpx is None:
                self.tpx = TPExchange(group, h.device)
            return TPMlpFn.apply(h, self.w1, self.w2, self.tpx)
        return tp_mlp_reference(h, self.w1, self.w2, group)
