"""Work partitioning for more than one GPU.

The hot path shards without a data-path exchange: ciphertext columns, token blocks, limbs and
polynomials are independent units.  A single PCMM is split by COLUMN RANGE so that all limbs of
a column stay on one GPU and the fused rescale by the last limb needs nothing from a peer; the
only collective is the optional gather of the output for a consumer that wants it whole.
"""
import torch
import torch.distributed as dist

TILE = 32     # column granularity of ckks_b200_pcmm_ppmm


def column_ranges(width, world, tile=TILE):
    """Split [0, width) into `world` contiguous ranges whose bounds are multiples of `tile`
    (the last range ends at `width`).  Ranges differ by at most one tile; some may be empty
    when there are fewer tiles than ranks."""
    tiles = (width + tile - 1) // tile
    base, extra = divmod(tiles, world)
    out, t0 = [], 0
    for r in range(world):
        t1 = t0 + base + (1 if r < extra else 0)
        out.append((min(t0 * tile, width), min(t1 * tile, width)))
        t0 = t1
    return out


def unit_ranges(count, world):
    """Split `count` independent units (limbs, polynomials, token blocks) into contiguous ranges."""
    base, extra = divmod(count, world)
    out, u0 = [], 0
    for r in range(world):
        u1 = u0 + base + (1 if r < extra else 0)
        out.append((u0, u1))
        u0 = u1
    return out


def gather_output(out_full, ranges, group=None):
    """All-gather the column ranges of a PCMM output.

    out_full: [M][limbs][C] tensor on every rank in which only this rank's columns
    (ranges[rank]) are valid.  On return every rank holds all columns.  Ranges may be ragged:
    slices are padded to the widest one for the collective."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    wmax = max(c1 - c0 for c0, c1 in ranges)
    M, limbs, _ = out_full.shape
    mine = torch.zeros((M, limbs, wmax), dtype=out_full.dtype, device=out_full.device)
    c0, c1 = ranges[rank]
    mine[:, :, :c1 - c0] = out_full[:, :, c0:c1]
    parts = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(parts, mine, group=group)
    for r, (a, b) in enumerate(ranges):
        if r != rank and b > a:
            out_full[:, :, a:b] = parts[r][:, :, :b - a]
    return out_full
