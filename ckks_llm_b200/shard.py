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


def row_owner_ranges(rows, world):
    """Rows [begin, end) of every rank when the output rows of a column-sharded PCMM are dealt to owners: equal
    contiguous runs of ceil(rows / world) rounded up to a multiple of 32, the rule of ckks_b200_pcmm_set_row_owners."""
    per = ((rows + world - 1) // world + 31) // 32 * 32
    return [(min(per * r, rows), min(per * (r + 1), rows)) for r in range(world)]


def scatter_rows_to_owners(out_full, col_ranges, group=None):
    """The exchange the PCMM's row-owner epilogue performs with peer stores, as point-to-point messages: for
    transports without peer memory (and for tests on CPU ranks).  out_full: [M][limbs][C] on every rank with this
    rank's columns valid for ALL rows; on return this rank holds all columns of ITS rows (other rows are
    unchanged).  Every rank sends (world-1)/world of its part and receives as much."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    rows = row_owner_ranges(out_full.shape[0], world)
    c0, c1 = col_ranges[rank]
    r0, r1 = rows[rank]
    sends, recvs, ops = [], [], []
    for peer in range(world):
        if peer == rank:
            continue
        p0, p1 = rows[peer]
        a, b = col_ranges[peer]
        if p1 > p0 and c1 > c0:
            buf = out_full[p0:p1, :, c0:c1].contiguous()
            sends.append(buf)
            ops.append(dist.P2POp(dist.isend, buf, peer, group))
        if r1 > r0 and b > a:
            buf = torch.empty((r1 - r0, out_full.shape[1], b - a), dtype=out_full.dtype, device=out_full.device)
            recvs.append((a, b, buf))
            ops.append(dist.P2POp(dist.irecv, buf, peer, group))
    if ops:
        for req in dist.batch_isend_irecv(ops):
            req.wait()
    for a, b, buf in recvs:
        out_full[r0:r1, :, a:b] = buf
    return rows[rank]


def gather_output(out_full, ranges, group=None, rows_per_step=None):
    """All-gather the column ranges of a PCMM output.

    out_full: [M][limbs][C] tensor on every rank in which only this rank's columns
    (ranges[rank]) are valid.  On return every rank holds all columns.  Ranges may be ragged:
    slices are padded to the widest one for the collective.  rows_per_step bounds the staging
    memory: the rows are gathered that many at a time (default: all at once)."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    wmax = max(c1 - c0 for c0, c1 in ranges)
    M, limbs, _ = out_full.shape
    step = M if not rows_per_step else max(1, min(M, int(rows_per_step)))
    c0, c1 = ranges[rank]
    mine = torch.zeros((step, limbs, wmax), dtype=out_full.dtype, device=out_full.device)
    parts = torch.empty((world * step, limbs, wmax), dtype=out_full.dtype, device=out_full.device)   # rank r at rows r*step..
    for m0 in range(0, M, step):
        m1 = min(M, m0 + step)
        n = m1 - m0
        mine[:n, :, :c1 - c0] = out_full[m0:m1, :, c0:c1]
        dist.all_gather_into_tensor(parts, mine, group=group)
        for r, (a, b) in enumerate(ranges):
            if r != rank and b > a:
                out_full[m0:m1, :, a:b] = parts[r * step:r * step + n, :, :b - a]
    return out_full


def gather_limbs(limb_major, limb_ranges, group=None):
    """All-gather the limbs of a batch of polynomials transformed limb by limb on different ranks.

    limb_major: [limbs][polys][N] tensor on every rank (limb-major, so that a rank's limbs are one contiguous block)
    in which only this rank's limbs (limb_ranges[rank]) are valid.  On return every rank holds all limbs.  Equal ranges
    go out as one in-place all-gather; ragged ones are padded to the largest."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    sizes = [b - a for a, b in limb_ranges]
    if len(set(sizes)) == 1 and limb_ranges[0][0] == 0 and sizes[0] * world == limb_major.shape[0]:
        a, b = limb_ranges[rank]
        dist.all_gather_into_tensor(limb_major, limb_major[a:b], group=group)
        return limb_major
    wmax = max(sizes)
    mine = torch.zeros((wmax,) + tuple(limb_major.shape[1:]), dtype=limb_major.dtype, device=limb_major.device)
    a, b = limb_ranges[rank]
    mine[:b - a] = limb_major[a:b]
    parts = torch.empty((world * wmax,) + tuple(limb_major.shape[1:]), dtype=limb_major.dtype, device=limb_major.device)
    dist.all_gather_into_tensor(parts, mine, group=group)
    for r, (x, y) in enumerate(limb_ranges):
        if r != rank and y > x:
            limb_major[x:y] = parts[r * wmax:r * wmax + (y - x)]
    return limb_major


def open_peer_buffers(t, group=None):
    """Maps the other ranks' copies of a CUDA tensor into this process for kernels on this rank's GPU.

    Every rank passes its own tensor `t` (same shape everywhere).  The ranks exchange the CUDA IPC handles of the
    allocations behind their tensors and each opens the others' with its own GPU current.  Returns
    ({rank: device address of that rank's tensor}, [base addresses to hand to close_peer_buffers]).  The owners must
    keep their tensors alive for as long as anybody uses the mappings."""
    import ctypes as C
    from . import capi
    lib = capi.load()
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    info = t.untyped_storage()._share_cuda_()          # (device, handle bytes, size, offset of the storage in its allocation, ...)
    handle = bytes(info[1])
    if len(handle) == 66:                              # torch prefixes the 64-byte handle with a version and a kind byte
        if handle[1:2] == b"e":
            raise RuntimeError("the tensor's memory is an expandable segment, not a cudaMalloc block: no IPC memory handle")
        handle = handle[2:]
    if len(handle) != 64:
        raise RuntimeError(f"unexpected CUDA IPC handle length {len(handle)}")
    meta = (handle, int(info[3]) + t.storage_offset() * t.element_size())
    metas = [None] * world
    dist.all_gather_object(metas, meta, group=group)
    addrs, bases = {}, []
    for r in range(world):
        if r == rank:
            continue
        handle, offset = metas[r]
        base = C.c_void_p()
        capi.check(lib.ckks_b200_ipc_open(t.device.index, handle, C.byref(base)))
        bases.append(base.value)
        addrs[r] = base.value + offset
    return addrs, bases


def close_peer_buffers(device_index, bases):
    from . import capi
    lib = capi.load()
    for b in bases:
        capi.check(lib.ckks_b200_ipc_close(device_index, b))
