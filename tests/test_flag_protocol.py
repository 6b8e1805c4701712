"""Replay of the device-side signalling protocols under adversarial schedules, on the CPU.

The kernels synchronise ranks through monotone epoch words in peer memory (``csrc/comm.cu``: rank r release-stores
its epoch into word r of every peer's flag row and acquire-spins on its own row until every word has reached the
epoch, comparing with a signed 32-bit difference) and through monotone arrival counters (``csrc/gemm_ag.cuh``). Here
the same rules run as interleaved atomic steps chosen by hypothesis, and the safety properties are checked: nobody
leaves barrier k before everybody entered it, data written before a barrier is seen after it, a slow rank several
epochs behind never lets a fast rank through, and the comparison survives the 32-bit wrap of the epoch."""
import numpy as np
import pytest
from hypothesis import given, settings, strategies as st

MASK = 0xFFFFFFFF


def _behind(seen: int, epoch: int) -> bool:
    """``static_cast<int32_t>(seen - epoch) < 0`` of the kernels."""
    d = (seen - epoch) & MASK
    return d >= 0x80000000


class Rank:
    def __init__(self, r, world, epoch0):
        self.r, self.world, self.epoch = r, world, epoch0
        self.phase, self.k = "work", 0          # work -> store(q = 0..world-1) -> spin -> work ...
        self.q = 0
        self.entered, self.left = [], []


def _run(world, rounds, schedule, epoch0):
    flags = np.full((world, world), epoch0 & MASK, dtype=np.uint64)      # flags[r][q]: q's epoch as seen by r
    data = np.zeros(world, dtype=np.int64)                               # "payload" each rank writes before a barrier
    ranks = [Rank(r, world, epoch0 & MASK) for r in range(world)]
    seen_after = [[] for _ in range(world)]
    steps = 0
    it = iter(schedule)
    while any(x.k < rounds for x in ranks):
        steps += 1
        assert steps < 200_000, "no progress: the protocol dead-locked"
        try:
            r = next(it) % world
        except StopIteration:
            r = steps % world                   # after the adversarial prefix: round robin until everybody is done
        x = ranks[r]
        if x.k >= rounds:
            continue
        if x.phase == "work":
            data[r] = x.k + 1                   # the write that the barrier has to publish
            x.epoch = (x.epoch + 1) & MASK
            x.entered.append(steps)
            x.phase, x.q = "store", 0
        elif x.phase == "store":                # one release store per step: peers may run in between
            flags[x.q][r] = x.epoch
            x.q += 1
            if x.q == world:
                x.phase = "spin"
        else:
            if all(not _behind(int(flags[r][q]), x.epoch) for q in range(world)):
                seen_after[r].append(data.copy())
                x.left.append(steps)
                x.k += 1
                x.phase = "work"
    return ranks, seen_after


@settings(max_examples=150, deadline=None)
@given(world=st.integers(2, 8), rounds=st.integers(1, 5), schedule=st.lists(st.integers(0, 7), max_size=400),
       epoch0=st.sampled_from([0, 1, 0x7FFFFFFE, 0xFFFFFFFD]))
def test_epoch_barrier_is_safe_under_any_interleaving(world, rounds, schedule, epoch0):
    ranks, seen_after = _run(world, rounds, schedule, epoch0)
    for k in range(rounds):
        last_entry = max(x.entered[k] for x in ranks)
        assert all(x.left[k] > last_entry for x in ranks), "a rank left the barrier before every rank had entered it"
        for r in range(world):
            assert (seen_after[r][k] >= k + 1).all(), "a write made before the barrier is not visible after it"


def test_fast_rank_cannot_lap_a_slow_one():
    """One rank runs ahead as far as the protocol lets it (it is scheduled exclusively): it must stop inside its
    first barrier, because the others have not arrived."""
    ranks, _ = _run(3, 1, [0] * 50 + [1, 2] * 50, epoch0=0)
    assert ranks[0].left[0] > max(ranks[1].entered[0], ranks[2].entered[0])


@settings(max_examples=100, deadline=None)
@given(n_chunks=st.integers(1, 6), schedule=st.lists(st.integers(0, 1), max_size=200), call=st.integers(1, 5))
def test_arrival_counter_consumer_never_reads_a_chunk_early(n_chunks, schedule, call):
    """All-gather -> GEMM: the producer copies chunk c, then bumps the monotone arrival word to ``call``; the consumer's
    tile for chunk c waits until the word has reached the value of this call. Counters are never reset between calls,
    so a value left by an earlier call must not satisfy the wait."""
    arrived = [call - 1] * n_chunks            # state after the previous call
    copied = [False] * n_chunks
    pc, cc = 0, 0                              # producer / consumer progress
    it = iter(schedule)
    guard = 0
    while cc < n_chunks:
        guard += 1
        assert guard < 10_000
        who = next(it, guard % 2)
        if who == 0 and pc < 2 * n_chunks:
            c, half = divmod(pc, 2)
            if half == 0:
                copied[c] = True
            else:
                arrived[c] = call
            pc += 1
        elif who == 1:
            if arrived[cc] - call >= 0:
                assert copied[cc], "consumer passed the wait before the chunk was copied"
                cc += 1


@pytest.mark.parametrize("world,rows", [(2, 32400), (4, 16200), (8, 8100), (8, 1000)])
def test_reduce_scatter_tile_rotation_spreads_the_owners(world, rows):
    """The reduce-scatter GEMM of rank r starts at the 256-row tile that holds the first row of rank r + 1 and walks
    the tiles cyclically (``GemmParams::tm_rot``). Restated here: every rank still visits every tile once, ends on its
    own rows, and at any position of the walk the ranks push to (almost always) different owners, so no GPU's
    ingress carries everybody's traffic at once, which the unrotated order did."""
    M = world * rows
    m_tiles = (M + 255) // 256
    order = {}
    for r in range(world):
        rot = (((r + 1) % world) * rows) // 256
        order[r] = [(tm + rot) % m_tiles for tm in range(m_tiles)]
        assert sorted(order[r]) == list(range(m_tiles))
        first_owner = min(order[r][0] * 256, M - 1) // rows
        assert first_owner in ((r + 1) % world, r)                      # a tile that straddles the boundary may start in r
        assert (order[r][-1] * 256) // rows in (r, (r + 1) % world, (r - 1) % world) or world == 2

    def owner(tile):
        return min(tile * 256 + 128, M - 1) // rows                    # owner of the tile's middle row
    rotated = sum(len({owner(order[r][i]) for r in range(world)}) for i in range(m_tiles)) / m_tiles
    plain = sum(len({owner(i) for _ in range(world)}) for i in range(m_tiles)) / m_tiles
    assert plain == 1.0 and rotated > 0.9 * world


def test_folded_four_value_block_reduction_lane_algebra():
    """``block_sum4_shfl`` (csrc/elementwise.cu) restated with arrays for lanes: lanes that differ in bit 4 split the four
    values two and two, lanes that differ in bit 3 one and one, three more exchanges finish the warp sum; value k of
    warp w lands in slot k * 8 + w and one more three-step fold per slot row gives every lane all four block totals."""
    rng = np.random.default_rng(0)
    n_warps = 6
    s = rng.standard_normal((n_warps, 32, 4))                      # [warp, lane, value]
    lanes = np.arange(32)
    red = np.zeros(32)
    for w in range(n_warps):
        v = s[w]
        b4, b3 = (lanes & 16) != 0, (lanes & 8) != 0
        a0, a1 = np.where(b4, v[:, 2], v[:, 0]), np.where(b4, v[:, 3], v[:, 1])
        g0, g1 = np.where(b4, v[:, 0], v[:, 2]), np.where(b4, v[:, 1], v[:, 3])
        a0, a1 = a0 + g0[lanes ^ 16], a1 + g1[lanes ^ 16]
        c, d = np.where(b3, a1, a0), np.where(b3, a0, a1)
        c = c + d[lanes ^ 8]
        for o in (4, 2, 1):
            c = c + c[lanes ^ o]
        for lane in (0, 8, 16, 24):
            red[(lane >> 3) * 8 + w] = c[lane]
    t = red.copy()
    for o in (4, 2, 1):
        t = t + t[lanes ^ o]
    totals = np.array([t[j * 8] for j in range(4)])
    assert np.allclose(totals, s.sum(axis=(0, 1)))
    assert all(np.allclose(t[j * 8:(j + 1) * 8], totals[j]) for j in range(4))     # every lane of a group holds it


@pytest.mark.parametrize("rows,K,grid", [(32400, 1536, 148), (8100, 1536, 148), (1000, 512, 148), (129, 8, 148),
                                         (16200, 4096, 132)])
def test_all_gather_copier_slices_cover_the_chunk_in_aligned_pieces(rows, K, grid):
    """``ag_push_chunk`` (csrc/gemm_ag.cuh): every CTA moves one contiguous slice of this rank's chunk in pieces of at
    most 16 KB; bulk copies need 16-byte aligned addresses and sizes. Restated: the slices are disjoint, cover the
    chunk exactly, and every piece starts and ends on a 16-byte boundary."""
    total = rows * K * 2
    assert total % 16 == 0                                             # checked on the host before the launch
    per = ((total // 16 + grid - 1) // grid) * 16
    covered = 0
    for b in range(grid):
        b0, b1 = per * b, min(total, per * (b + 1))
        if b0 >= b1:
            continue
        assert b0 == covered and b0 % 16 == 0
        pos = b0
        while pos < b1:
            n = min(16384, b1 - pos)
            assert n % 16 == 0 and pos % 16 == 0 and 0 < n <= 16384
            pos += n
        covered = b1
    assert covered == total


def test_reduce_scatter_stage_pitch_is_conflict_free_for_quarter_warps():
    """Linear staging of the reduce-scatter epilogue: 32 rows of 256 bytes at a pitch of 272 bytes. A 16-byte access of
    lane l to chunk c of its own row touches banks ((272 l + 16 c) / 4 + 0..3) mod 32; the eight lanes of a quarter
    warp (one shared-memory wavefront for 128-bit accesses) must fall into disjoint banks, and every row must start
    on a 16-byte boundary for the bulk copy."""
    pitch = 272
    assert pitch % 16 == 0
    for c in range(16):
        for q in range(4):
            banks = set()
            for lane in range(8 * q, 8 * q + 8):
                first = ((pitch * lane + 16 * c) // 4) % 32
                banks.update((first + k) % 32 for k in range(4))
            assert len(banks) == 32
