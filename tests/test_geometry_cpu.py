"""Host-side geometry that the CUDA kernels rely on, checked on CPU against the layout library."""
import numpy as np
import torch

from aeris_gb_b200.models import layout as LY
from aeris_gb_b200.ops import attention as A
from aeris_gb_b200.ops import diffusion as DF


def _row_to_pixel(g: DF.TokGeom, row: int):
    """Python restatement of the device function row_to_pixel (csrc/diffusion.cu)."""
    rps = g.nwy_loc * g.nwx_loc * g.n_local
    b, r = divmod(row, rps)
    w, tok = divmod(r, g.n_local)
    seq = g.sp_rank * g.n_local + tok
    iy, ix = divmod(seq, g.ws_x)
    wy, wx = divmod(w, g.nwx_loc)
    return b, wy * g.ws_y + iy, wx * g.ws_x + ix


def test_token_geometry_matches_layout():
    """Row r of a rank's unshifted token stream is the pixel that the layout library says it is, for WP and SP."""
    for wp, sp in (((1, 1), 1), ((2, 2), 1), ((1, 2), 2), ((2, 1), 4)):
        grid = LY.Grid(32, 64, 8, 8, wp[0], wp[1], sp)
        for rank in range(grid.n_ranks):
            g = DF.make_geom(grid, 2, rank)
            ys, xs = LY.rank_pixels(grid, (0, 0), rank)
            assert g.rows == 2 * ys.size
            for row in (0, 1, ys.size // 2, ys.size - 1, ys.size, 2 * ys.size - 1):
                b, y, x = _row_to_pixel(g, row)
                assert b == row // ys.size
                assert (g.y0 + y, g.x0 + x) == (ys[row % ys.size], xs[row % ys.size]), (wp, sp, rank, row)


def test_head_padding_round_trip():
    T, H, d, dp = 10, 3, 32, 64
    qkv = torch.randn(T, 3 * H * d)
    p = A._pad_heads(qkv, 3, H, d, dp)
    assert p.shape == (T, 3 * H * dp)
    assert torch.equal(A._unpad_heads(p, 3, H, d, dp), qkv)
    assert p.view(T, 3, H, dp)[..., d:].abs().max() == 0
    assert A._kernel_dim(64) == 64 and A._kernel_dim(128) == 128 and A._kernel_dim(32) == 64 and A._kernel_dim(96) == 128


def test_gather_tables_are_permutations_of_the_other_layout():
    """Going to the shifted layout and back through the two tables is the identity, over all ranks."""
    grid = LY.Grid(32, 64, 8, 8, 2, 2)
    n = grid.n_ranks
    src = [torch.arange(grid.tokens_per_rank).float().unsqueeze(1) + 1000 * r for r in range(n)]
    shifted = [LY.apply_gather_reference(LY.gather_table(grid, (0, 0), grid.half_shift(), r), src) for r in range(n)]
    back = [LY.apply_gather_reference(LY.gather_table(grid, grid.half_shift(), (0, 0), r), shifted) for r in range(n)]
    for r in range(n):
        assert torch.equal(back[r], src[r])
    assert 0.0 < LY.halo_fraction(grid) < 0.5
    assert np.isclose(LY.halo_fraction(LY.Grid(32, 64, 8, 8)), 0.0)


def test_rope_2d_is_a_relative_rotation():
    """Rotating q at position a and k at position b leaves q.k a function of (a - b) per axis, and the inverse flag
    undoes the rotation."""
    from aeris_gb_b200.models import oracle as O
    ws_y, ws_x, d = 4, 6, 16
    cos, sin = O.rope_2d_cache(ws_y, ws_x, d)
    assert cos.shape == (ws_y * ws_x, d // 2)
    g = torch.Generator().manual_seed(0)
    q, k = torch.randn(d, generator=g), torch.randn(d, generator=g)
    L = ws_y * ws_x
    Q = O.apply_rope_2d(q.expand(L, d), cos, sin)
    K = O.apply_rope_2d(k.expand(L, d), cos, sin)
    S = Q @ K.t()
    pos = lambda y, x: y * ws_x + x
    assert torch.allclose(S[pos(1, 2), pos(0, 1)], S[pos(3, 5), pos(2, 4)], atol=1e-5)     # same offset (1, 1)
    assert torch.allclose(S[pos(0, 0), pos(0, 0)], q @ k, atol=1e-5)
    assert not torch.allclose(S[pos(1, 2), pos(0, 1)], S[pos(1, 2), pos(0, 0)], atol=1e-4)
    x = torch.randn(2, 3, L, d, generator=g)
    assert torch.allclose(O.apply_rope_2d(O.apply_rope_2d(x, cos, sin), cos, sin, inverse=True), x, atol=1e-5)


def test_hi_lo_split_makes_bf16_products_fp32_accurate():
    """The fp32 ends of the network run on the bf16 tensor cores by splitting both operands into a bf16 value and a
    bf16 remainder; the three products hi*hi + hi*lo + lo*hi (fp32 accumulation) then match the fp32 product to about
    2^-16, against 2^-8 for plain bf16 operands."""
    from aeris_gb_b200.models.fused_io import _split
    g = torch.Generator().manual_seed(0)
    a, w = torch.randn(64, 144, generator=g), torch.randn(70, 144, generator=g)
    exact = a.double() @ w.double().t()
    a_hi, a_lo = (t.float() for t in _split(a))
    w_hi, w_lo = (t.float() for t in _split(w))
    assert torch.equal(a_hi + a_lo, (a_hi + a_lo).to(torch.float32)) and (a - (a_hi + a_lo)).abs().max() < 2e-5
    plain = (a_hi @ w_hi.t()).double()
    split = (a_hi @ w_hi.t() + a_hi @ w_lo.t() + a_lo @ w_hi.t()).double()
    err_plain = ((plain - exact).norm() / exact.norm()).item()
    err_split = ((split - exact).norm() / exact.norm()).item()
    assert err_split < 3e-5 and err_plain > 50 * err_split


def test_separable_position_tables_rebuild_the_full_encoding():
    from aeris_gb_b200.models import oracle as O
    C, H, W = 10, 6, 9
    ty, tx = O.positional_tables(C, H, W)
    full = O.positional_encoding_2d(C, H, W)
    ch = ty.shape[1]
    both = torch.cat([ty.unsqueeze(1).expand(H, W, ch), tx.unsqueeze(0).expand(H, W, ch)], dim=-1)[..., :C]
    assert torch.allclose(full, both)
