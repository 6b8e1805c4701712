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
