"""Index arithmetic of the fused expert-parallel kernels, restated in Python and checked for every
world size the layer supports (1, 2, 4, 8) without a GPU:

  * the dispatch send (copy role of the GEMM kernel): every (chunk, destination, expert, slot) row is moved
    exactly once, lands inside the receive buffer, no two items write the same bytes, and the row counts
    the senders add to a destination's 128-row block flags sum to the block's size;
  * the flag gate of GEMM 1 and the de-quantiser's unit list: every 128-row block a tile reads has a flag,
    the segment-interleaved tile order is a permutation, and the units cover every row once, in tile order;
  * the push epilogue: destination rows are unique and inside the combine buffer, and the number of
    arrivals each (chunk, source) flag receives equals what the host helper ``gemm_push_arrivals`` tells
    the receiver to wait for.

The formulas mirror ``csrc/kernels/gemm_tcgen05.cu`` (``copy_role``, ``dequant_role``, ``mtile_coord``, the
producer's gate, the push epilogue) and ``ops/fused_moe.py``."""

import itertools

import pytest

from planmoe_b200.ops import native

BM = 128            # accumulator rows per CTA
GATE_BLOCK = 128    # rows per arrival flag
COPY_BYTES, MIN_SLOT = 65536, 4096


def _copy_items(W, my_rank, E_l, C, d, M, grid, quant=False, local_first=True):
    """(cta, dest, group, first row in the destination group, rows, [dst byte offset of each row]) per item."""
    Cc = C // d
    wire = M + 16 if quant else M * 2                        # bytes of a row, at the source and on the wire
    slot = MIN_SLOT
    while slot < wire:
        slot *= 2
    lanes = COPY_BYTES // slot // 2                          # rows per item: half of the slots (two alternating sets)
    per_seg = (Cc + lanes - 1) // lanes
    n_items = d * E_l * per_seg * W
    out = []
    for cta in range(grid):
        for item in range(cta, n_items, grid):
            if not local_first or W == 1:
                rr = item % W
                t = item // W
                sub, g = t % per_seg, t // per_seg
            else:                                            # chunk by chunk: own rows of every group, then the others
                per_chunk_loc = E_l * per_seg
                j, t = divmod(item, per_chunk_loc * W)
                if t < per_chunk_loc:
                    rr = W - 1
                else:
                    t -= per_chunk_loc
                    rr = t % (W - 1)
                    t //= W - 1
                sub, el = t % per_seg, t // per_seg
                g = j * E_l + el
            r = (my_rank + 1 + rr) % W
            row0 = sub * lanes
            nrows = min(lanes, Cc - row0)
            dsts = [((g * W + my_rank) * Cc + row0 + i) * wire for i in range(nrows)]
            out.append((cta, r, g, my_rank * Cc + row0, nrows, dsts))
    return out, wire


@pytest.mark.parametrize("local_first", [False, True])
@pytest.mark.parametrize("quant", [False, True])
@pytest.mark.parametrize("W,E_l,C,d,M", [(1, 2, 8192, 1, 2048), (2, 2, 4096, 4, 2048), (4, 2, 2048, 2, 2048),
                                        (8, 2, 1024, 4, 2048), (8, 8, 320, 1, 1024), (8, 1, 96, 2, 4096),
                                        (4, 3, 40, 1, 72), (2, 2, 260, 1, 8192)])
def test_dispatch_send_covers_every_slot_once(W, E_l, C, d, M, quant, local_first):
    if quant and M % 16:
        pytest.skip("int8 rows need a multiple of 16 elements")
    grid = 148
    Cc = C // d
    R = W * Cc
    nblk = (R + GATE_BLOCK - 1) // GATE_BLOCK
    flags = {}                                               # (dest, group, block) -> rows added by all senders
    for my_rank in range(W):
        items, wire = _copy_items(W, my_rank, E_l, C, d, M, grid, quant, local_first)
        if local_first and W > 1:                            # a chunk's own-rank items come before its other items
            per_cta = {}
            for cta, r, g, first, nrows, dsts in items:
                per_cta.setdefault(cta, []).append((g // E_l, r != my_rank))
            for seq in per_cta.values():
                assert seq == sorted(seq)
        buf_bytes = d * E_l * W * Cc * wire                  # receive buffer of one destination rank
        seen = set()
        rows_to = {}
        for cta, r, g, first, nrows, dsts in items:
            for dst in dsts:
                assert 0 <= dst and dst + wire <= buf_bytes
                assert (r, dst) not in seen, "two items write the same bytes"
                seen.add((r, dst))
            rows_to[(r, g)] = rows_to.get((r, g), 0) + nrows
            left, f = nrows, first                            # the signal: rows split over the blocks they touch
            while left > 0:
                blk = f // GATE_BLOCK
                n = min(left, (blk + 1) * GATE_BLOCK - f)
                assert blk < nblk
                flags[(r, g, blk)] = flags.get((r, g, blk), 0) + n
                f += n
                left -= n
        for r in range(W):
            for g in range(d * E_l):
                assert rows_to.get((r, g), 0) == Cc, (r, g)  # every destination gets all my rows of every group
    for r in range(W):
        for g in range(d * E_l):
            for blk in range(nblk):
                assert flags.get((r, g, blk), 0) == min(GATE_BLOCK, R - blk * GATE_BLOCK), (r, g, blk)


def _mtile_coord(ordinal, mt_count, perm_w, perm_q, perm_local, gpc, my_rank):
    """(group, m-tile) of the ordinal-th m-tile in consumption order (mtile_coord of the kernel)."""
    if perm_q <= 1:
        return divmod(ordinal, mt_count)
    if not perm_local:
        g, l = divmod(ordinal, mt_count)
        return g, (l % perm_w) * perm_q + l // perm_w
    chunk, u = divmod(ordinal, gpc * mt_count)
    if u < gpc * perm_q:
        el, k = divmod(u, perm_q)
        mt = my_rank * perm_q + k
    else:
        u -= gpc * perm_q
        others = perm_w - 1
        el, l = divmod(u, others * perm_q)
        src = (my_rank + 1 + l % others) % perm_w
        mt = src * perm_q + l // others
    return chunk * gpc + el, mt


@pytest.mark.parametrize("perm_local", [0, 1])
@pytest.mark.parametrize("W,E_l,C,d,cg", [(1, 2, 8192, 1, 2), (2, 2, 4096, 4, 2), (4, 2, 2048, 2, 2), (8, 2, 1024, 4, 2),
                                         (8, 2, 1024, 1, 2), (8, 2, 1024, 8, 2), (8, 8, 320, 1, 2), (2, 2, 48, 2, 1)])
def test_tile_order_and_dequant_units_cover_every_block(W, E_l, C, d, cg, perm_local):
    Cc = C // d
    R = W * Cc                                               # rows per (chunk, expert) group
    tile_rows = BM * cg
    mt_count = (R + tile_rows - 1) // tile_rows
    perm_w, perm_q = 0, 0
    if W > 1 and Cc > tile_rows and Cc % tile_rows == 0 and W * Cc == R:
        perm_w, perm_q = W, Cc // tile_rows
    groups = d * E_l
    my_rank = W // 2
    coords = [_mtile_coord(i, mt_count, perm_w, perm_q, perm_local, E_l, my_rank) for i in range(groups * mt_count)]
    assert sorted(coords) == [(g, mt) for g in range(groups) for mt in range(mt_count)]     # a permutation
    assert [g // E_l for g, _ in coords] == sorted(g // E_l for g, _ in coords)              # chunks stay in order
    if perm_q > 1 and not perm_local:                        # first tile of every source before any second tile
        assert [mt // perm_q for _, mt in coords[:W]] == list(range(W))
    if perm_q > 1 and perm_local:                            # a chunk starts with this rank's segment of every group
        head = coords[:E_l * perm_q]
        assert all(mt // perm_q == my_rank for _, mt in head) and sorted({g for g, _ in head}) == list(range(E_l))
        nxt = coords[E_l * perm_q:E_l * perm_q + W - 1]      # then tile 0 of every other source, right neighbour first
        assert [mt // perm_q for _, mt in nxt] == [(my_rank + 1 + i) % W for i in range(W - 1)]
    order = [mt for g, mt in coords if g == 0]
    nblk = (R + GATE_BLOCK - 1) // GATE_BLOCK
    # de-quantiser units: 32 rows each, listed in tile order; every row exactly once, inside a flagged block
    units_per_block = GATE_BLOCK // 32
    covered = []
    for u in range(mt_count * cg * units_per_block):
        sub = u % units_per_block
        t = u // units_per_block
        b = t % cg
        mt = order[t // cg]                                  # the units of group 0, in its tile order
        blk = mt * cg + b
        row0 = blk * GATE_BLOCK + sub * 32
        if row0 >= R:
            continue
        assert blk < nblk
        covered += list(range(row0, min(row0 + 32, R)))
    assert sorted(covered) == list(range(R))
    # the producer of a CTA tile waits for the one block its 128 rows lie in
    for mt in range(mt_count):
        for cr in range(cg):
            m0 = mt * tile_rows + cr * BM
            if m0 < R:
                assert m0 // GATE_BLOCK < nblk and m0 % GATE_BLOCK == 0


@pytest.mark.parametrize("W,E_l,C,d", [(1, 2, 8192, 1), (2, 2, 4096, 4), (4, 2, 2048, 2), (8, 2, 1024, 4),
                                      (8, 2, 1024, 8), (8, 8, 320, 1), (2, 2, 48, 2)])
def test_gate_flags_of_the_unfused_send_cover_the_rows_a_tile_reads(W, E_l, C, d):
    Cc = C // d
    R = W * Cc                                               # rows per (chunk, expert) group
    for m0 in range(0, R, BM):
        last = min(m0 + BM, R) - 1
        s_lo, s_hi = m0 // Cc, last // Cc
        owners = {m // Cc for m in range(m0, last + 1)}      # source rank of every row of the tile
        assert owners == set(range(s_lo, s_hi + 1))
        assert s_hi < W


@pytest.mark.parametrize("W,E_l,C,d,N", [(1, 2, 8192, 1, 2048), (2, 2, 4096, 4, 2048), (4, 2, 2048, 2, 2048),
                                        (8, 2, 1024, 4, 2048), (8, 8, 320, 1, 1024), (2, 2, 48, 2, 64),
                                        (4, 1, 100, 1, 320)])
def test_push_epilogue_rows_and_arrivals(W, E_l, C, d, N):
    lib = native.lib()
    Cc = C // d
    R = W * Cc
    BN = 256
    nt = (N + BN - 1) // BN
    for my_rank in {0, W - 1}:
        arrivals = {}                                        # (dest rank, chunk) -> arrivals from my launch
        rows_seen = {}
        for g in range(d * E_l):
            chunk, el = divmod(g, E_l)
            for m0 in range(0, R, BM):
                last = min(m0 + BM, R) - 1
                for m in range(m0, last + 1):
                    s, cc = divmod(m, Cc)
                    drow = (my_rank * E_l + el) * C + chunk * Cc + cc
                    assert 0 <= drow < W * E_l * C           # inside rank s's combine buffer [E_global * C, N]
                    assert (s, drow) not in rows_seen
                    rows_seen[(s, drow)] = True
                for s in range(m0 // Cc, last // Cc + 1):
                    arrivals[(s, chunk)] = arrivals.get((s, chunk), 0) + nt      # one arrival per (m-tile, n-tile)
        for s in range(W):
            want = lib.gemm_push_arrivals(E_l, R, N, Cc, s)  # what the receiver adds to its expected count
            for chunk in range(d):
                assert arrivals.get((s, chunk), 0) == want, (s, chunk)
        assert len(rows_seen) == d * E_l * R
        # the bulk-store form of the epilogue needs each 32-row slice inside one source rank's block
        if Cc % 32 == 0:
            for m0 in range(0, R, 32):
                assert m0 // Cc == (m0 + 31) // Cc


def test_routing_bounds_check_accepts_consistent_and_rejects_corrupt():
    import pytest
    import torch
    from planmoe_b200.ops.fused_moe import check_routing_bounds
    S, E, C, K = 6, 2, 3, 1
    idx = torch.tensor([[0, 1, 0, 0, 1, 0]], dtype=torch.int32)
    loc = torch.tensor([[0, 0, 1, 2, 1, 3]], dtype=torch.int32)          # the last pick is dropped (slot 3 >= C)
    slot_map = torch.tensor([0, 2, 3, 1, 4, -1], dtype=torch.int32)      # expert 0: tokens 0, 2, 3; expert 1: 1, 4, empty
    check_routing_bounds(idx, loc, slot_map, S, E, C, K)
    bad = slot_map.clone(); bad[5] = 5                                   # an owner nobody claims
    with pytest.raises(AssertionError):
        check_routing_bounds(idx, loc, bad, S, E, C, K)
    bad = idx.clone(); bad[0, 2] = 2                                     # expert out of range
    with pytest.raises(AssertionError):
        check_routing_bounds(bad, loc, slot_map, S, E, C, K)
    bad = slot_map.clone(); bad[1] = 3; bad[2] = 2                       # two picks swapped: they no longer own their slots
    with pytest.raises(AssertionError):
        check_routing_bounds(idx, loc, bad, S, E, C, K)
