"""Host-side multi-rank logic on CPU: two gloo ranks split a PPMM by column range, compute
their shards with the oracle, gather, and must reproduce the unsharded result."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import helpers as H
from ckks_llm_b200 import params, shard


def test_column_ranges_cover_and_align():
    for width, world in [(65664, 8), (4160, 2), (96, 8), (67584, 8), (33, 2)]:
        rs = shard.column_ranges(width, world)
        assert rs[0][0] == 0 and rs[-1][1] == width
        for (a, b), (c, d) in zip(rs, rs[1:]):
            assert b == c
        for a, b in rs:
            assert a % 32 == 0 and (b % 32 == 0 or b == width) and a <= b
        widths = [b - a for a, b in rs if b > a]
        assert max(widths) - min(widths) <= 32 + 31
    assert shard.unit_ranges(20, 8) == [(0, 3), (3, 6), (6, 9), (9, 12), (12, 14), (14, 16), (16, 18), (18, 20)]


def test_row_owner_ranges_follow_the_library_rule():
    """Equal runs of ceil(M / world) rounded up to 32 rows (the rule of ckks_b200_pcmm_row_owner_range, which the GPU test
    of the row-owner epilogue checks against the library)."""
    assert shard.row_owner_ranges(4096, 8) == [(512 * r, 512 * (r + 1)) for r in range(8)]
    assert shard.row_owner_ranges(150, 3) == [(0, 64), (64, 128), (128, 150)]
    assert shard.row_owner_ranges(40, 2) == [(0, 32), (32, 40)]
    assert shard.row_owner_ranges(20, 4) == [(0, 20), (20, 20), (20, 20), (20, 20)]


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import oracle as O
    q = params.ntt_primes(50, 1 << 13, 3)
    rng = np.random.default_rng(0)                 # same inputs on both ranks
    M, K, N1, k = 40, 16, 32, 2                    # width 96: three tiles over two ranks (ragged); rows 0..31 and 32..39
    Cw = (k + 1) * N1
    W = rng.uniform(-1, 1, (M, K)).astype(np.float32)
    X = np.stack([H.uniform_residues(rng, q, (Cw,)) for _ in range(K)])
    ranges = shard.column_ranges(Cw, world)
    c0, c1 = ranges[rank]
    out = torch.zeros((M, len(q), Cw), dtype=torch.int64)
    part = O.ppmm(W, np.ascontiguousarray(X[:, :, c0:c1]), q, float(1 << 40))
    out[:, :, c0:c1] = torch.from_numpy(part.view(np.int64))
    full = O.ppmm(W, X, q, float(1 << 40))
    # rows to their owners: this rank ends with all columns of its rows and nothing new elsewhere
    own = out.clone()
    r0, r1 = shard.scatter_rows_to_owners(own, ranges)
    ok_rows = bool(np.array_equal(own[r0:r1].numpy().view(np.uint64), full[r0:r1]))
    mask = torch.ones_like(own, dtype=torch.bool)
    mask[r0:r1] = False
    ok_rest = bool(torch.equal(own[mask], out[mask]))
    shard.gather_output(out, ranges)
    ret[rank] = bool(np.array_equal(out.numpy().view(np.uint64), full)) and ok_rows and ok_rest
    dist.destroy_process_group()


def test_two_ranks_column_sharded_ppmm_gloo():
    world = 2
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(180)
        assert p.exitcode == 0
    assert all(ret[r] for r in range(world))


def _limb_worker(rank, world, port, limbs, ret):
    """Every rank transforms its own limbs of the same batch (with the CPU restatement standing in for the GPU) and
    the limbs are gathered: all ranks must end with the transform of the whole batch."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import oracle as O
    N, polys = 256, 3
    q = params.ntt_primes(40, 2 * N, limbs)
    T = O.NttTables(N, q)
    rng = np.random.default_rng(5)
    data = np.stack([np.stack([rng.integers(0, qi, N, dtype=np.uint64) for qi in q]) for _ in range(polys)])   # [poly][limb][N]
    want = data.copy()
    O.ntt_batch(want, T, 0, 0, polys, limbs, limbs)
    ranges = shard.unit_ranges(limbs, world)
    a, b = ranges[rank]
    mine = data.copy()
    if b > a:
        O.ntt_batch(mine, T, a, a, polys, b - a, limbs)          # limbs [a, b) of every polynomial
    limb_major = torch.from_numpy(np.ascontiguousarray(mine.transpose(1, 0, 2)).view(np.int64)).clone()
    for i in range(limbs):
        if not a <= i < b:
            limb_major[i] = -1                                    # what this rank did not compute is not valid
    shard.gather_limbs(limb_major, ranges)
    got = limb_major.numpy().view(np.uint64).transpose(1, 0, 2)
    ret[rank] = bool(np.array_equal(got, want))
    dist.destroy_process_group()


@pytest.mark.parametrize("limbs", [4, 5])
def test_two_ranks_limb_sharded_transform_gloo(limbs):
    """Equal limb ranges take the in-place all-gather, ragged ones (5 limbs on 2 ranks) the padded one."""
    world = 2
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_limb_worker, args=(r, world, port, limbs, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(180)
        assert p.exitcode == 0
    assert all(ret[r] for r in range(world))
