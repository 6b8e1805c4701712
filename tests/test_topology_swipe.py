"""Rank grid, groups and SWiPe routing (pure CPU)."""
import numpy as np
import pytest

from aeris_gb_b200.parallel import swipe as S
from aeris_gb_b200.parallel.topology import ProcessGrid


def test_grid_coords_and_groups():
    g = ProcessGrid(world_size=2 * 2 * 2 * 3 * 4, PP=3, SP=4, WP_Y=2, WP_X=2)
    assert g.DP == 2
    for r in range(g.used):
        c = g.coords(r)
        assert g.rank_of(c.dp, c.wp_y, c.wp_x, c.pp, c.sp) == r
    # SP fastest, then PP
    assert g.coords(1).sp == 1 and g.coords(4).pp == 1
    assert len(g.sp_ranks(0)) == 4 and len(g.pp_ranks(0)) == 3 and len(g.weight_ranks(0)) == 2 * 4 * 4
    for kind, n in (("sp", 4), ("pp", 3), ("wp", 4), ("dp", 2), ("weight", 32)):
        lists = g.all_group_lists(kind)
        assert all(len(l) == n for l in lists)
        assert sorted(sum(lists, [])) == list(range(g.used))      # a partition of the ranks
    assert g.stage_heads() == [0, 4, 8]


def test_grid_rejects_too_few_ranks():
    with pytest.raises(AssertionError):
        ProcessGrid(world_size=8, PP=4, SP=4)


@pytest.mark.parametrize("SP", [1, 2, 4, 12])
@pytest.mark.parametrize("WP", [(1, 1), (2, 2), (2, 4)])
def test_swipe_layout_is_a_partition_and_returns_to_identity(SP, WP):
    g = S.SwipeGeometry(H=48, W=96, ws_y=12, ws_x=12, WP_Y=WP[0], WP_X=WP[1], SP=SP)
    img = np.arange(g.H * g.W).reshape(g.H, g.W, 1)
    for shifted in (False, True):
        seen = np.concatenate([S.tile_sample(img, g, shifted, y, x, s).ravel()
                               for y in range(g.WP_Y) for x in range(g.WP_X) for s in range(SP)])
        assert sorted(seen.tolist()) == list(range(g.H * g.W))
    # plain -> shifted -> plain via the routes reproduces every rank's rows
    def move(bufs, a, b):
        new = {k: np.empty_like(v) for k, v in bufs.items()}
        for (y, x, s), buf in bufs.items():
            for dst, (srow, drow) in S.route(g, a, b, y, x, s).items():
                new[dst][drow] = buf[srow]
        return new
    bufs = {(y, x, s): S.tile_sample(img, g, False, y, x, s)
            for y in range(g.WP_Y) for x in range(g.WP_X) for s in range(SP)}
    shifted = move(bufs, False, True)
    for k, v in shifted.items():
        assert np.array_equal(v, S.tile_sample(img, g, True, *k))
    back = move(shifted, True, False)
    for k, v in back.items():
        assert np.array_equal(v, bufs[k])


def test_shifted_windows_are_windows_of_the_rolled_image():
    g = S.SwipeGeometry(H=24, W=48, ws_y=12, ws_x=12, WP_Y=2, WP_X=2, SP=1)
    img = np.arange(g.H * g.W).reshape(g.H, g.W, 1)
    rolled = np.roll(img, shift=(-6, -6), axis=(0, 1))
    for y in range(2):
        for x in range(2):
            assert np.array_equal(S.tile_sample(img, g, True, y, x, 0), S.tile_sample(rolled, g, False, y, x, 0))


@pytest.mark.parametrize("shift_up_next", [True, False])
def test_sp12_routes_match_the_reference_table(shift_up_next):
    g = S.SwipeGeometry(H=48, W=48, ws_y=12, ws_x=12, WP_Y=2, WP_X=2, SP=12)
    src_shifted = not shift_up_next     # odd stage (plain layout) sends "up" into the shifted layout
    for y in range(2):
        for x in range(2):
            for sp in range(12):
                r = S.route(g, src_shifted, not src_shifted, y, x, sp)
                assert len(r) == 1, "with SP = 12 every rank has exactly one pipeline peer"
                (dst,) = r.keys()
                assert dst == S.reference_next_rank_sp12(y, x, sp, 2, 2, shift_up_next)
                s2 = S.recv_plan(g, src_shifted, not src_shifted, *dst)
                assert (y, x, sp) in s2


def test_stage_shift_pattern():
    assert [S.stage_is_shifted(p, 10) for p in range(10)] == [False, False, True, False, True, False, True, False, True, False]
