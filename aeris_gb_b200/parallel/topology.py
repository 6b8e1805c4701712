"""Process grid and communication groups: ranks are laid out as a 5-D grid ``(DP, WP_Y, WP_X, PP, SP)`` with SP fastest
and PP next (reference: ``grid_init``, src/aeris/parallelism/parallel_engine.py:294-313). Group membership is computed
as plain rank lists (testable without any process group); :meth:`ProcessGrid.build_groups` turns them into
``torch.distributed`` groups.

Groups (reference lines in parentheses): ``sp`` = same (dp, wp, pp) (:379); ``pp`` = same (dp, wp, sp) (:391);
``weight`` = every rank of one pipeline stage, i.e. all of DP x WP x SP (:400-402), the group gradients are reduced
over; ``wp`` = same (dp, pp, sp) (window-parallel peers, used by the halo exchange and result gathers); ``dp``;
``pipe`` = for every pair of neighbouring pipeline stages two 2-rank groups, one per direction of travel (the reference
creates pairwise ``pp_comm_group_{prev,next}`` groups, :425-451): activations go down one, gradients come up the other,
so the point-to-point operations of each communicator all flow one way and match in issue order.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np


@dataclass(frozen=True)
class Coords:
    dp: int
    wp_y: int
    wp_x: int
    pp: int
    sp: int


class ProcessGrid:
    def __init__(self, world_size: int, PP: int = 1, SP: int = 1, WP_Y: int = 1, WP_X: int = 1, DP: int | None = None):
        per_replica = WP_Y * WP_X * PP * SP
        assert per_replica <= world_size, \
            f"not enough ranks for WP {WP_Y}x{WP_X}, PP {PP}, SP {SP}: need {per_replica}, have {world_size}"
        self.DP = DP if DP is not None else world_size // per_replica
        assert self.DP * per_replica <= world_size
        self.WP_Y, self.WP_X, self.PP, self.SP = WP_Y, WP_X, PP, SP
        self.world_size = world_size
        self.used = self.DP * per_replica
        self.grid = np.arange(self.used).reshape(self.DP, WP_Y, WP_X, PP, SP)

    # ---- coordinates ------------------------------------------------------------------------------------------
    def coords(self, rank: int) -> Coords:
        assert 0 <= rank < self.used, f"rank {rank} is outside the grid of {self.used} ranks"
        dp, y, x, pp, sp = np.unravel_index(rank, self.grid.shape)
        return Coords(int(dp), int(y), int(x), int(pp), int(sp))

    def rank_of(self, dp: int, wp_y: int, wp_x: int, pp: int, sp: int) -> int:
        return int(self.grid[dp, wp_y % self.WP_Y, wp_x % self.WP_X, pp, sp])

    def is_first_stage(self, rank: int) -> bool:
        return self.coords(rank).pp == 0

    def is_last_stage(self, rank: int) -> bool:
        return self.coords(rank).pp == self.PP - 1

    # ---- rank lists -------------------------------------------------------------------------------------------
    def sp_ranks(self, rank: int) -> list[int]:
        c = self.coords(rank)
        return self.grid[c.dp, c.wp_y, c.wp_x, c.pp, :].flatten().tolist()

    def pp_ranks(self, rank: int) -> list[int]:
        c = self.coords(rank)
        return self.grid[c.dp, c.wp_y, c.wp_x, :, c.sp].flatten().tolist()

    def wp_ranks(self, rank: int) -> list[int]:
        c = self.coords(rank)
        return self.grid[c.dp, :, :, c.pp, c.sp].flatten().tolist()

    def replica_ranks(self, rank: int) -> list[int]:
        """WP x SP ranks that together hold one sample at one pipeline stage (row-major over (wp_y, wp_x, sp))."""
        c = self.coords(rank)
        return self.grid[c.dp, :, :, c.pp, :].flatten().tolist()

    def dp_ranks(self, rank: int) -> list[int]:
        c = self.coords(rank)
        return self.grid[:, c.wp_y, c.wp_x, c.pp, c.sp].flatten().tolist()

    def weight_ranks(self, rank: int) -> list[int]:
        c = self.coords(rank)
        return self.grid[:, :, :, c.pp, :].flatten().tolist()

    def tp_ranks(self, rank: int) -> list[int]:
        """The ranks that split the MLP weights of a tensor-parallel model between them: ranks that hold different
        token rows of the same sample, i.e. the SP group when SP > 1, else the WP x SP ranks of the sample."""
        return self.sp_ranks(rank) if self.SP > 1 else self.replica_ranks(rank)

    def tp_ortho_ranks(self, rank: int) -> list[int]:
        """The ranks of the weight group that hold the same tensor-parallel shard as ``rank``."""
        pos = self.tp_ranks(rank).index(rank)
        return [q for q in self.weight_ranks(rank) if self.tp_ranks(q).index(q) == pos]

    def stage_heads(self) -> list[int]:
        """One rank per pipeline stage (dp = wp = sp = 0): the ranks that write checkpoints (:1229)."""
        return self.grid[0, 0, 0, :, 0].flatten().tolist()

    def pipe_pairs(self) -> list[tuple[int, int]]:
        """(rank of stage s, rank of stage s + 1) for every pipeline link of the grid, in a fixed global order."""
        out = []
        for r in range(self.used):
            c = self.coords(r)
            if c.pp + 1 < self.PP:
                out.append((r, self.rank_of(c.dp, c.wp_y, c.wp_x, c.pp + 1, c.sp)))
        return out

    def all_group_lists(self, kind: str) -> list[list[int]]:
        fn = {"sp": self.sp_ranks, "pp": self.pp_ranks, "wp": self.wp_ranks, "dp": self.dp_ranks,
              "weight": self.weight_ranks, "replica": self.replica_ranks, "tp": self.tp_ranks,
              "tp_ortho": self.tp_ortho_ranks}[kind]
        seen, out = set(), []
        for r in range(self.used):
            g = tuple(fn(r))
            if g not in seen:
                seen.add(g)
                out.append(list(g))
        return out

    # ---- torch.distributed groups -----------------------------------------------------------------------------
    def build_groups(self, rank: int, kinds=("sp", "pp", "wp", "dp", "weight", "replica", "pipe"),
                     backend: str | None = None) -> dict:
        """Creates every group of the requested kinds on every rank (``new_group`` is collective over the world) and
        returns this rank's group of each kind. Groups of size 1 are returned as ``None``. Kind ``pipe`` yields the
        keys ``down_next`` / ``up_next`` (links to the next stage), ``down_prev`` / ``up_prev`` and ``result`` (last
        stage to first stage)."""
        import torch.distributed as dist
        mine = {}
        for kind in kinds:
            if kind == "pipe":
                for lo, hi in self.pipe_pairs():
                    for direction in ("down", "up"):
                        g = dist.new_group([lo, hi], backend=backend)
                        if rank == lo:
                            mine[f"{direction}_next"] = g
                        elif rank == hi:
                            mine[f"{direction}_prev"] = g
                if self.PP > 1:      # last stage -> first stage: results of the inference schedule
                    for r in range(self.used):
                        c = self.coords(r)
                        if c.pp == 0:
                            last = self.rank_of(c.dp, c.wp_y, c.wp_x, self.PP - 1, c.sp)
                            g = dist.new_group([r, last], backend=backend)
                            if rank in (r, last):
                                mine["result"] = g
                continue
            for ranks in self.all_group_lists(kind):
                if len(ranks) == 1:
                    if rank in ranks:
                        mine[kind] = None
                    continue
                g = dist.new_group(ranks, backend=backend)
                if rank in ranks:
                    mine[kind] = g
        return mine

    def describe(self) -> str:
        return (f"ProcessGrid(DP={self.DP}, WP={self.WP_Y}x{self.WP_X}, PP={self.PP}, SP={self.SP}, "
                f"used {self.used} of {self.world_size} ranks)")
