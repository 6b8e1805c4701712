"""Numerics of every CUDA kernel against a plain PyTorch fp32 reference of the same op."""
import math

import pytest
import torch

from conftest import rel_err

pytestmark = pytest.mark.gpu
DEV = "cuda"
TOL = 6e-3  # bf16 outputs of fp32-accumulated products


@pytest.fixture(autouse=True)
def _seed():
    torch.manual_seed(0)


@pytest.mark.parametrize("M,N,K", [(256, 256, 128), (1000, 384, 192), (2048, 1536, 1536)])
@pytest.mark.parametrize("a_t,b_t", [(False, False), (True, False), (False, True), (True, True)])
def test_gemm_layouts(M, N, K, a_t, b_t):
    from aeris_gb_b200.ops import gemm as G
    a = torch.randn(M, K, device=DEV).bfloat16()
    b = torch.randn(N, K, device=DEV).bfloat16()
    ref = a.float() @ b.float().t()
    out = G.gemm(a.t().contiguous() if a_t else a, b.t().contiguous() if b_t else b, a_t=a_t, b_t=b_t)
    assert rel_err(out, ref) < TOL
    out128 = G.gemm(a.t().contiguous() if a_t else a, b.t().contiguous() if b_t else b, a_t=a_t, b_t=b_t, bn=128)
    assert rel_err(out128, ref) < TOL


@pytest.mark.parametrize("M,N,K", [(300, 256, 128), (4096, 1024, 512)])
def test_gemm_epilogues(M, N, K):
    from aeris_gb_b200.ops import gemm as G
    a = torch.randn(M, K, device=DEV).bfloat16()
    b = torch.randn(N, K, device=DEV).bfloat16()
    ref = a.float() @ b.float().t()
    assert rel_err(G.gemm(a, b, epi=G.EPI_STORE_F32), ref) < 1e-5
    acc0 = torch.randn(M, N, device=DEV)
    for ks in (1, 2, 3):
        o = acc0.clone()
        G.gemm(a, b, out=o, epi=G.EPI_ACC_F32, k_splits=ks)
        assert rel_err(o, ref + acc0) < 1e-5
    F = N // 2
    sref = torch.nn.functional.silu(ref[:, :F]) * ref[:, F:]
    assert rel_err(G.gemm(a, b, epi=G.EPI_SWIGLU), sref) < TOL
    raw = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    act = G.gemm(a, b, epi=G.EPI_SWIGLU_BOTH, aux=raw)
    assert rel_err(act, sref) < TOL and rel_err(raw, ref) < TOL
    # fused SwiGLU backward: product = d(act) [M, F], u given, d(u) out (in place)
    u = torch.randn(M, 2 * N, device=DEV).bfloat16()
    ur = u.float().requires_grad_(True)
    (torch.nn.functional.silu(ur[:, :N]) * ur[:, N:]).backward(ref)
    du = u.clone()
    G.gemm(a, b, out=du, epi=G.EPI_SWIGLU_BWD, resid=du)
    assert rel_err(du, ur.grad) < TOL
    x = torch.randn(M, N, device=DEV).bfloat16()
    g = torch.randn(1, N, device=DEV)
    aux = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    o = G.gemm(a, b, epi=G.EPI_GATE_RESID, resid=x, gate=g, aux=aux)
    assert rel_err(o, x.float() + g * ref) < TOL and rel_err(aux, ref) < TOL


@pytest.mark.parametrize("nw,N,H,d", [(2, 64, 2, 64), (3, 256, 2, 64), (3, 900, 4, 64), (2, 900, 2, 128), (2, 100, 1, 64),
                                        (2, 64, 4, 32), (2, 900, 2, 32), (1, 3600, 2, 128), (1, 3600, 2, 64)])
def test_attention_fwd_bwd(nw, N, H, d):
    from aeris_gb_b200.ops import attention as A
    qkv = torch.randn(nw * N, 3 * H * d, device=DEV).bfloat16()
    go = torch.randn(nw * N, H * d, device=DEV).bfloat16()
    o, lse = A.attn_fwd(qkv, nw, N, H, d)
    dqkv = A.attn_bwd(qkv, o, go, lse, nw, N, H, d)
    x = qkv.float().requires_grad_(True)
    ref = A.attn_reference(x, nw, N, H, d)
    ref.backward(go.float())
    assert rel_err(o, ref) < TOL
    HD = H * d
    for i in range(3):
        assert rel_err(dqkv[:, i * HD:(i + 1) * HD], x.grad[:, i * HD:(i + 1) * HD]) < 8e-3
    q, k, _ = qkv.float().view(nw, N, 3, H, d).permute(2, 0, 3, 1, 4)
    lref = torch.logsumexp((q @ k.transpose(-1, -2)) / math.sqrt(d), -1) / math.log(2)
    assert (lse - lref).abs().max().item() < 1e-3


@pytest.mark.parametrize("N,d", [(900, 64), (900, 128), (320, 64)])
def test_attention_fwd_rising_scores(N, d):
    """Scores that grow along the key sequence by far more than 2^8: the forward kernel must raise its reference
    maximum (and rescale its TMEM accumulator) many times, in full and in partial tiles."""
    from aeris_gb_b200.ops import attention as A
    nw, H = 4, 3
    g = torch.Generator(device=DEV).manual_seed(3)
    qkv = torch.randn(nw, N, 3, H, d, device=DEV, generator=g)
    ramp = torch.linspace(0.2, 6.0, N, device=DEV).view(1, N, 1, 1)
    qkv[:, :, 0] *= 3.0
    qkv[:, :, 1] *= ramp                       # later keys score higher (and lower) than earlier ones
    qkv = qkv.reshape(nw * N, 3 * H * d).bfloat16()
    o, lse = A.attn_fwd(qkv, nw, N, H, d)
    ref = A.attn_reference(qkv.float(), nw, N, H, d)
    assert torch.isfinite(o.float()).all()
    assert rel_err(o, ref) < 1.5e-2
    q, k, _ = qkv.float().view(nw, N, 3, H, d).permute(2, 0, 3, 1, 4)
    lref = torch.logsumexp((q @ k.transpose(-1, -2)) / math.sqrt(d), -1) / math.log(2)
    assert (lse - lref).abs().max().item() < 2e-2


@pytest.mark.parametrize("variant,mode,d", [(0, 0, 64), (2, 0, 64), (-1, 1, 64), (2, 1, 64), (-1, 2, 64), (-1, 1, 128)])
def test_attention_fwd_variants(variant, mode, d):
    """The forward kernel with two-wide fp32 softmax arithmetic, part of the exponentials on the polynomial exp2, and
    the probabilities kept in tensor memory: plain and strongly rising scores (partial last tile included) against
    the fp32 formulation, same tolerances as the default kernel."""
    from aeris_gb_b200.ops import attention as A
    A.set_fwd_variant(variant, mode)
    try:
        nw, N, H = 3, 900, 4
        qkv = torch.randn(nw * N, 3 * H * d, device=DEV).bfloat16()
        o, lse = A.attn_fwd(qkv, nw, N, H, d)
        ref = A.attn_reference(qkv.float(), nw, N, H, d)
        assert rel_err(o, ref) < TOL
        q, k, _ = qkv.float().view(nw, N, 3, H, d).permute(2, 0, 3, 1, 4)
        lref = torch.logsumexp((q @ k.transpose(-1, -2)) / math.sqrt(d), -1) / math.log(2)
        assert (lse - lref).abs().max().item() < 1e-3
        g = torch.Generator(device=DEV).manual_seed(3)
        r = torch.randn(nw, N, 3, H, d, device=DEV, generator=g)
        r[:, :, 0] *= 3.0
        r[:, :, 1] *= torch.linspace(0.2, 6.0, N, device=DEV).view(1, N, 1, 1)
        r = r.reshape(nw * N, 3 * H * d).bfloat16()
        o2, _ = A.attn_fwd(r, nw, N, H, d)
        assert torch.isfinite(o2.float()).all()
        assert rel_err(o2, A.attn_reference(r.float(), nw, N, H, d)) < 1.5e-2
    finally:
        A.set_fwd_variant(-1, 0)


def test_attention_bwd_rising_scores():
    """Backward on scores that spread over many powers of two along the key sequence (sharp softmax rows): the
    recomputed probabilities come from the forward's log-sum-exp, so nothing may overflow or lose the small terms."""
    from aeris_gb_b200.ops import attention as A
    nw, N, H, d = 2, 900, 2, 64
    g = torch.Generator(device=DEV).manual_seed(5)
    r = torch.randn(nw, N, 3, H, d, device=DEV, generator=g)
    r[:, :, 0] *= 2.0
    r[:, :, 1] *= torch.linspace(0.2, 4.0, N, device=DEV).view(1, N, 1, 1)
    qkv = r.reshape(nw * N, 3 * H * d).bfloat16()
    go = torch.randn(nw * N, H * d, device=DEV, generator=g).bfloat16()
    o, lse = A.attn_fwd(qkv, nw, N, H, d)
    dqkv = A.attn_bwd(qkv, o, go, lse, nw, N, H, d)
    x = qkv.float().requires_grad_(True)
    A.attn_reference(x, nw, N, H, d).backward(go.float())
    assert torch.isfinite(dqkv.float()).all()
    HD = H * d
    for i in range(3):
        assert rel_err(dqkv[:, i * HD:(i + 1) * HD], x.grad[:, i * HD:(i + 1) * HD]) < 2e-2


@pytest.mark.parametrize("D", [128, 1536])
@pytest.mark.parametrize("mode", [0, 1])
def test_modnorm_fwd_bwd(D, mode):
    from aeris_gb_b200.ops import elementwise as E
    rows, eps = 777, 1e-3
    x = torch.randn(rows, D, device=DEV).bfloat16()
    sc, sh = torch.randn(D, device=DEV) * 0.3, torch.randn(D, device=DEV) * 0.3
    w = (1 + 0.1 * torch.randn(D, device=DEV)).bfloat16()
    dh = torch.randn(rows, D, device=DEV).bfloat16()
    dres = torch.randn(rows, D, device=DEV).bfloat16()

    def ref_fn(xv, scv, shv, wv):
        def rms(v):
            return v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps) * wv
        return rms(xv * (1 + scv) + shv) if mode == 0 else rms(xv) * (1 + scv) + shv

    xr, scr, shr, wr = [t.float().requires_grad_(True) for t in (x, sc, sh, w)]
    href = ref_fn(xr, scr, shr, wr)
    href.backward(dh.float())
    h = E.modnorm_fwd(x, sc, sh, w, mode=mode, eps=eps)
    assert rel_err(h, href) < TOL
    dx = torch.empty_like(x)
    dsc, dsh, dw = [torch.zeros(D, device=DEV) for _ in range(3)]
    E.modnorm_bwd(x, dh, dres, sc, sh, w, mode=mode, eps=eps, dx=dx, dscale=dsc, dshift=dsh, dw=dw)
    assert rel_err(dx, xr.grad + dres.float()) < TOL
    assert rel_err(dsc, scr.grad) < 2e-3 and rel_err(dsh, shr.grad) < 2e-3 and rel_err(dw, wr.grad) < 2e-3


def test_modnorm_gather_and_gather_rows():
    from aeris_gb_b200.ops import elementwise as E
    D, rows = 256, 500
    src = torch.randn(rows, D, device=DEV).bfloat16()
    perm = torch.randperm(rows, device=DEV).to(torch.int32)
    w = torch.ones(D, device=DEV).bfloat16()
    xo = torch.empty_like(src)
    h = E.modnorm_fwd(src, None, None, w, mode=0, eps=1e-3, gather_idx=perm, peer_ptrs=[src.data_ptr()], x_out=xo)
    g = src[perm.long()]
    assert torch.equal(xo, g)
    ref = g.float() * torch.rsqrt(g.float().pow(2).mean(-1, keepdim=True) + 1e-3)
    assert rel_err(h, ref) < TOL
    out = torch.empty_like(src)
    E.gather_rows(perm, [src.data_ptr()], out)
    assert torch.equal(out, g)


@pytest.mark.parametrize("heads,d", [(4, 64), (2, 128)])
def test_rope_kernel_matches_fp32_rotation_and_its_inverse(heads, d):
    """In-place 2-D rotary embedding of the q and k sections of a fused qkv tensor against the fp32 formula; v stays
    untouched; the inverse rotation restores q and k to bf16 rounding."""
    from aeris_gb_b200.models import oracle as O
    from aeris_gb_b200.ops import elementwise as E
    ws, nw = (6, 10), 3
    L = ws[0] * ws[1]
    cos, sin = O.rope_2d_cache(ws[0], ws[1], d, 10_000.0, DEV)
    qkv = torch.randn(nw * L, 3 * heads * d, device=DEV).bfloat16()
    v5 = qkv.float().view(nw, L, 3, heads, d)
    ref = v5.clone()
    for i in (0, 1):
        ref[:, :, i] = O.apply_rope_2d(v5[:, :, i].permute(0, 2, 1, 3), cos, sin).permute(0, 2, 1, 3)
    got = qkv.clone()
    E.rope_qk_(got, cos.float().contiguous(), sin.float().contiguous(), L, heads, d)
    assert rel_err(got, ref.view(nw * L, -1)) < TOL
    assert torch.equal(got.view(nw, L, 3, heads, d)[:, :, 2], qkv.view(nw, L, 3, heads, d)[:, :, 2])
    E.rope_qk_(got, cos.float().contiguous(), sin.float().contiguous(), L, heads, d, inverse=True)
    assert rel_err(got, qkv) < 2 * TOL


def test_swiglu_and_gate_helpers():
    from aeris_gb_b200.ops import elementwise as E
    rows, F = 333, 512
    u = torch.randn(rows, 2 * F, device=DEV).bfloat16()
    d = torch.randn(rows, F, device=DEV).bfloat16()
    ur = u.float().requires_grad_(True)
    ref = torch.nn.functional.silu(ur[:, :F]) * ur[:, F:]
    ref.backward(d.float())
    assert rel_err(E.swiglu_fwd(u), ref) < TOL
    assert rel_err(E.swiglu_bwd(u, d), ur.grad) < TOL
    R, C = 128, 256
    W = torch.randn(R, C, device=DEV).bfloat16()
    g = torch.randn(R, device=DEV)
    assert rel_err(E.scale_rows(W, g), W.float() * g[:, None]) < TOL
    Gm = torch.randn(R, C, device=DEV)
    dW0 = torch.randn(R, C, device=DEV)
    dW, dg = dW0.clone(), torch.zeros(R, device=DEV)
    Gc = Gm.clone()
    E.gate_grad_finalize(Gc, W, g, dW, dg)
    assert rel_err(dW, dW0 + g[:, None] * Gm) < 1e-5
    assert rel_err(dg, (W.float() * Gm).sum(1)) < 1e-4
    assert Gc.abs().max().item() == 0


def test_adamw_matches_torch():
    from aeris_gb_b200.ops import elementwise as E
    n = 10_001
    p0 = torch.randn(n, device=DEV)
    ref_p = torch.nn.Parameter(p0.clone())
    opt = torch.optim.AdamW([ref_p], lr=1e-2, betas=(0.85, 0.9), eps=1e-8, weight_decay=0.2)
    master, m, v = p0.clone(), torch.zeros(n, device=DEV), torch.zeros(n, device=DEV)
    wb = torch.empty(n, device=DEV, dtype=torch.bfloat16)
    ema = p0.clone()
    ema_ref = p0.clone()
    for step in range(1, 4):
        g = torch.randn(n, device=DEV)
        ref_p.grad = g.clone() * 0.5
        opt.step()
        ema_ref = ref_p.detach().lerp(ema_ref, 0.9)
        grad = g.clone()
        E.adamw(master, grad, m, v, wb, ema, None, lr=1e-2, betas=(0.85, 0.9), eps=1e-8, weight_decay=0.2,
                step=step, grad_scale=0.5, max_norm=0.0, ema_beta=0.9)
        assert grad.abs().max().item() == 0
    assert rel_err(master, ref_p.detach()) < 1e-5
    assert rel_err(ema, ema_ref) < 1e-5
    assert rel_err(wb, ref_p.detach()) < 5e-3
    # clipping through the global norm
    nsq = torch.zeros(1, device=DEV, dtype=torch.float64)
    g = torch.randn(n, device=DEV)
    E.sumsq(g, nsq)
    assert abs(nsq.item() - g.double().pow(2).sum().item()) / nsq.item() < 1e-5


def test_bounded_wait_times_out_and_leaves_the_context_usable():
    """A device-side wait on a flag that nothing sets must give up after its limit and report it to the host."""
    import ctypes
    import time
    from aeris_gb_b200.ops import lib as L
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    t0 = time.perf_counter()
    rc = L.lib().aeris_wait_flag(L.ptr(flag), ctypes.c_uint(1), L.ptr(L.status_word()), ctypes.c_double(0.5),
                                 L.stream_ptr())
    assert rc == 0
    with pytest.raises(L.KernelError, match="peer signal"):
        L.check_status()
    assert 0.4 < time.perf_counter() - t0 < 5.0
    # the status word was cleared and the context still works
    a = torch.ones(1024, device=DEV)
    assert float((a * 2).sum()) == 2048.0
    flag.fill_(1)
    L.lib().aeris_wait_flag(L.ptr(flag), ctypes.c_uint(1), L.ptr(L.status_word()), ctypes.c_double(0.5), L.stream_ptr())
    L.check_status()
