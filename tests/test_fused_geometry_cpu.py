"""Index arithmetic of the fused expert-parallel kernels, restated in Python and checked for every
world size the layer supports (1, 2, 4, 8) without a GPU:

  * the dispatch send (copy role of the GEMM kernel): every (chunk, destination, expert, slot) row is moved
    exactly once, lands inside the receive buffer, and no two units write the same bytes;
  * the flag gate of GEMM 1: the source ranks a 128-row CTA tile waits for are exactly the ranks whose rows
    it reads;
  * the push epilogue: destination rows are unique and inside the combine buffer, and the number of
    arrivals each (chunk, source) flag receives equals what the host helper ``gemm_push_arrivals`` tells
    the receiver to wait for.

The formulas mirror ``csrc/kernels/gemm_tcgen05.cu`` (``copy_role``, the producer's gate, the push
epilogue) and ``ops/fused_moe.py``."""

import itertools

import pytest

from planmoe_b200.ops import native

BM = 128            # accumulator rows per CTA
SLOT = 4096         # bytes per bulk-copy unit


def _copy_units(W, my_rank, E_l, C, d, M, grid):
    """(cta, chunk, dest, row, piece, dst_byte_offset, bytes) for every unit the copy role moves."""
    Cc, row_bytes = C // d, M * 2
    rows = E_l * Cc
    pieces = (row_bytes + SLOT - 1) // SLOT
    out = []
    for cta in range(grid):
        my_rows = (rows - 1 - cta) // grid + 1 if cta < rows else 0
        units = W * my_rows * pieces
        for j in range(d):
            for u in range(units):
                piece = u % pieces
                k = (u // pieces) % my_rows
                rr = u // (pieces * my_rows)
                r = (my_rank + 1 + rr + cta) % W
                row = cta + k * grid
                el, cc = divmod(row, Cc)
                nbytes = min(SLOT, row_bytes - piece * SLOT)
                dst = ((((j * E_l + el) * W + my_rank) * Cc + cc) * row_bytes) + piece * SLOT
                out.append((cta, j, r, el, cc, piece, dst, nbytes))
    return out


@pytest.mark.parametrize("W,E_l,C,d,M", [(1, 2, 8192, 1, 2048), (2, 2, 4096, 4, 2048), (4, 2, 2048, 2, 2048),
                                        (8, 2, 1024, 4, 2048), (8, 8, 320, 1, 1024), (8, 1, 96, 2, 4096),
                                        (4, 3, 40, 1, 72)])
def test_dispatch_send_covers_every_slot_once(W, E_l, C, d, M):
    grid = 148
    Cc, row_bytes = C // d, M * 2
    buf_bytes = d * E_l * W * Cc * row_bytes                 # receive buffer of one destination rank
    for my_rank in {0, W - 1, W // 2}:
        seen = {}
        per_dest_chunk = {}
        for cta, j, r, el, cc, piece, dst, nbytes in _copy_units(W, my_rank, E_l, C, d, M, grid):
            assert 0 <= dst and dst + nbytes <= buf_bytes
            key = (r, dst)
            assert key not in seen, "two units write the same bytes"
            seen[key] = nbytes
            per_dest_chunk[(r, j)] = per_dest_chunk.get((r, j), 0) + nbytes
        # every destination receives, per chunk, all of my rows for its experts
        for r in range(W):
            for j in range(d):
                assert per_dest_chunk.get((r, j), 0) == E_l * Cc * row_bytes, (r, j)


@pytest.mark.parametrize("W,E_l,C,d", [(1, 2, 8192, 1), (2, 2, 4096, 4), (4, 2, 2048, 2), (8, 2, 1024, 4),
                                      (8, 2, 1024, 8), (8, 8, 320, 1), (2, 2, 48, 2)])
def test_gate_flags_cover_the_rows_a_tile_reads(W, E_l, C, d):
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
