"""The message tables of the stand-alone all-to-all algorithms, executed by a CPU model of the transfer
kernel: every algorithm on every (world, group) split must deliver the all-to-all permutation, signal
every flag exactly as often as the receivers expect, and name, for each message, the one flag that
guards all of the bytes it reads."""

import itertools
import os

import numpy as np
import pytest

from planmoe_b200.parallel import a2a


class _Blk:
    def __init__(self, offset, nbytes):
        self.offset, self.nbytes = offset, nbytes


class _Tr:
    def __init__(self, world, rank):
        self.world, self.rank = world, rank


def _plans(algo, W, L, n):
    """Per-rank (phases, arrivals) with one shared heap layout."""
    sizes = {'hetu': dict(a=L * W * n, b=L * W * n, c=W * n), 'dd': dict(a=W * n, b=W * n)}.get(algo, dict(a=W * n))
    bufs, off = {}, 0
    for k, v in sizes.items():
        bufs[k] = _Blk(off, v)
        off += v
    out = []
    for r in range(W):
        ch = a2a.A2AChannel.__new__(a2a.A2AChannel)
        ch.tr, ch.W, ch.me, ch.L = _Tr(W, r), W, r, L
        out.append(ch._plan(algo, 0, n, bufs))
    return out, bufs, off


@pytest.mark.parametrize("algo", ['flat', 'pipe', 'dd', 'hetu'])
@pytest.mark.parametrize("W,L", [(2, 1), (2, 2), (4, 2), (4, 4), (8, 4), (8, 2), (8, 8), (6, 3)])
def test_message_tables_deliver_all_to_all(algo, W, L):
    if algo == 'dd' and L in (1, W):
        pytest.skip("2DH degenerates to flat without two levels")
    n = 16
    plans, bufs, heap_bytes = _plans(algo, W, L, n)
    rng = np.random.default_rng(0)
    inputs = [rng.integers(0, 255, size=W * n, dtype=np.uint8) for _ in range(W)]
    heaps = [np.zeros(heap_bytes, dtype=np.uint8) for _ in range(W)]
    writer = [np.full(heap_bytes, -1, dtype=np.int64) for _ in range(W)]     # (logical phase << 16 | flag) that wrote a byte
    outs = [np.zeros(W * n, dtype=np.uint8) for _ in range(W)]
    flags = [dict() for _ in range(W)]                                       # rank -> {(logical, flag_idx): arrivals}
    n_phases = max(len(p[0]) for p in plans)
    arrivals = plans[0][1]
    for r in range(W):
        assert plans[r][1] == arrivals, "every rank must agree on the arrival counts"

    # Ranks do not all have the same number of phases (only leaders run some): order the launches by the
    # logical phase they signal / wait for, which is the order their data dependencies impose.
    def order_key(ph):
        return ph.logical if ph.logical is not None else 99

    for level in sorted({order_key(ph) for r in range(W) for ph in plans[r][0]}):
        for r in range(W):
            for ph in plans[r][0]:
                if order_key(ph) != level:
                    continue
                src = inputs[r] if ph.src == 'in' else heaps[r][bufs[ph.src].offset:]
                src_writer = None if ph.src == 'in' else writer[r][bufs[ph.src].offset:]
                if ph.wait_idx:
                    for f in ph.wait_idx:                                    # what the kernel would wait for
                        assert flags[r].get((ph.wait_phase, f), 0) == arrivals[ph.wait_phase], (algo, r, f)
                for dest, flag_idx, src_off, dst_off, nbytes, wait_one in ph.msgs:
                    if src_writer is not None:
                        tags = set(src_writer[src_off:src_off + nbytes].tolist())
                        assert -1 not in tags, "message reads bytes nobody wrote"
                        if wait_one >= 0:
                            assert wait_one in ph.wait_idx
                            assert tags == {(ph.wait_phase << 16) | wait_one}, (algo, r, tags, wait_one)
                    data = src[src_off:src_off + nbytes]
                    if dest < 0:
                        outs[r][dst_off:dst_off + nbytes] = data
                    else:
                        heaps[dest][dst_off:dst_off + nbytes] = data
                        writer[dest][dst_off:dst_off + nbytes] = (ph.logical << 16) | flag_idx
                        key = (ph.logical, flag_idx)
                        flags[dest][key] = flags[dest].get(key, 0) + 1
    for r in range(W):
        for s in range(W):
            assert np.array_equal(outs[r][s * n:(s + 1) * n], inputs[s][r * n:(r + 1) * n]), (algo, r, s)
