"""Block sharding of full fields over the WP grid, on the device.

The reference's WP-only stack loads every sample on rank 0 and scatters / gathers contiguous blocks over a gloo side
group with sleeps in between (src/aeris_wp_inference/era5.py:159-295). Here every rank slices its own block from the
sample (or reads its own file), and results are gathered with one NCCL all-gather."""
from __future__ import annotations

import torch
import torch.distributed as dist


def shard_block(field: torch.Tensor, wp: tuple[int, int], wp_rank: tuple[int, int]) -> torch.Tensor:
    """field [..., H, W, C] -> this rank's [..., H/wp_y, W/wp_x, C] block."""
    H, W = field.shape[-3], field.shape[-2]
    hb, wb = H // wp[0], W // wp[1]
    y, x = wp_rank
    return field[..., y * hb:(y + 1) * hb, x * wb:(x + 1) * wb, :].contiguous()


def gather_blocks(block: torch.Tensor, wp: tuple[int, int], group=None) -> torch.Tensor:
    """Inverse of :func:`shard_block` across the WP group (rank order: row-major over (wp_y, wp_x))."""
    n = wp[0] * wp[1]
    if n == 1:
        return block
    parts = [torch.empty_like(block) for _ in range(n)]
    dist.all_gather(parts, block.contiguous(), group=group)
    rows = [torch.cat(parts[y * wp[1]:(y + 1) * wp[1]], dim=-2) for y in range(wp[0])]
    return torch.cat(rows, dim=-3)
