"""Stand-alone all-to-all algorithms on the symmetric-heap transport (CUDA worlds).

Every algorithm is a short sequence of launches of one kernel (``csrc/kernels/a2a.cu``): wait on
local flags, copy a table of messages into peers' heaps, signal.  The tables carry all index
arithmetic, including the layout transforms of the hierarchical algorithms.

  flat   one message per peer, straight into the peer's receive buffer        (naive.cpp:11-27)
  pipe   the same messages issued as two concurrent launches on two streams:  (pipe.cpp:12-31)
         peers inside my group / peers outside it
  dd     2DH: exchange inside the group, then between groups                  (dd_comm.cpp:35-75)
  hetu   gather to the group leader, leaders exchange, leader scatters        (hetu.cpp:15-76)

"Group" = ``LOCAL_SIZE`` consecutive ranks (env; default all ranks).  Let W ranks, L per group,
N = W / L groups, n = bytes per (source, destination) pair.

Staging buffers and flags live in the symmetric heap and are double-buffered by call parity; flags
are cumulative arrival counters.  By default the result is copied out of the heap into an ordinary
tensor by the last launch, so callers own their output.  ``heap_out=True`` skips that copy: the last
launch only waits for the arrivals and the caller gets a view of the receive buffer in the heap, which
stays valid until this rank's next all-to-all of the same algorithm and parity, i.e. across exactly one
further call (peers can only overwrite it after this rank has entered the call after the next).

Variable-length payloads (``var_len=(len_off, len_base)``): every (source, destination) slice carries
its own size in a u32 at byte ``len_off`` and only ``len_base`` + that many bytes of the slice are
moved, at every hop of every algorithm, with no host read of the sizes (the LZ codec's wire).
Staging blocks are sized to the next power of two of the per-pair payload, so payload sizes that drift
reuse their block instead of growing the heap call by call.
"""

import os

import torch

from ..ops import native


def _local_size(world):
    ls = int(os.environ.get('LOCAL_SIZE', 0)) or world
    ls = min(ls, world)
    return ls if world % ls == 0 else world


class _Phase:
    """One launch: messages + the flags it waits on."""

    def __init__(self, msgs, wait_idx, src, wait_phase=None, stream=0, logical=None):
        # logical: index of the flag set this launch signals (None: signals nothing)
        self.msgs, self.wait_idx, self.src, self.wait_phase, self.stream = msgs, wait_idx, src, wait_phase, stream
        self.logical = logical


class A2AChannel:
    N_PHASES = 4

    def __init__(self, tr):
        self.tr = tr
        self.W, self.me = tr.world, tr.rank
        self.L = _local_size(self.W)
        self.calls = 0
        self.bufs = {}          # (algo, parity) -> dict(name -> HeapBlock), sized for `cap` bytes per pair
        self.arrived = {}       # (algo, parity, phase) -> cumulative arrivals expected per flag
        self.tables = {}
        self.side = None

    # -- resources ----------------------------------------------------------------------------
    def _ensure(self, algo, parity, n):
        """Staging buffers and flags of one (algorithm, call parity), sized for ``n`` bytes per pair.

        Buffers and their flags are carved out of ONE heap block: a kernel addresses both through the
        same table of peer base addresses, and a block never spans heap segments.  Flags are cumulative
        counters, and which flags a call advances depends on the algorithm (in the hierarchical ones
        only group leaders receive some phases), so every (algorithm, parity) owns its flags; a larger
        reallocation starts from fresh (zeroed) flags and zeroed counters."""
        key = (algo, parity)
        cur = self.bufs.get(key)
        if cur is not None and cur['cap'] >= n:
            return cur
        from .transport import HeapBlock
        W, L = self.W, self.L
        cap = 1 << 20
        while cap < n:
            cap <<= 1
        if algo == 'hetu':
            sizes = dict(a=L * W * cap, b=L * W * cap, c=W * cap)
        elif algo == 'dd':
            sizes = dict(a=W * cap, b=W * cap)
        else:
            sizes = dict(a=W * cap)
        sizes['flags'] = self.N_PHASES * W * 8
        total = sum((v + 1023) // 1024 * 1024 for v in sizes.values())
        blk = self.tr.alloc(total)
        cur, off = {}, blk.offset
        for k, v in sizes.items():
            cur[k] = HeapBlock(self.tr, blk.segment, off, v)
            off += (v + 1023) // 1024 * 1024
        cur['cap'] = cap
        self.bufs[key] = cur
        self.tables = {k: v for k, v in self.tables.items() if k[:2] != key}
        self.arrived = {k: v for k, v in self.arrived.items() if k[:2] != key}
        return cur

    def _flag_off(self, algo, parity, phase):
        return self.bufs[(algo, parity)]['flags'].offset + phase * self.W * 8

    def _flag_ptr(self, algo, parity, phase):
        return self.bufs[(algo, parity)]['flags'].local_ptr + phase * self.W * 8

    # -- message tables ---------------------------------------------------------------------------
    def _plan(self, algo, parity, n, bufs):
        """List of phases; a message is (dest, flag_idx, src_off, dst_off, bytes, wait_one): ``wait_one`` is the
        one flag of the waited phase this message's source bytes depend on (-1: all listed).  ``src`` names the
        buffer the offsets are relative to: 'in' (the caller's tensor) or a staging block."""
        W, L, me = self.W, self.L, self.me
        N = W // L
        mn, ml = me // L, me % L
        a = bufs['a']
        phases = []
        if algo in ('flat', 'pipe'):
            def push(peers, stream):
                return _Phase([(d, me, d * n, a.offset + me * n, n, -1) for d in peers], None, 'in', None, stream, 0)
            if algo == 'flat' or L == W or L == 1:
                phases.append(push(range(W), 0))
            else:
                intra = [d for d in range(W) if d // L == mn]
                inter = [d for d in range(W) if d // L != mn]
                phases.append(push(intra, 1))
                phases.append(push(inter, 2))
            # copy-out: the slice from source s only needs flag s, so it starts while others are in flight
            phases.append(_Phase([(-1, -1, s * n, s * n, n, s) for s in range(W)], list(range(W)), 'a', 0))
            arrivals = {0: 1}
        elif algo == 'dd':
            b = bufs['b']
            # phase 0: to local peer l' everything I send to local index l' of any group -> a[sl][dn]
            phases.append(_Phase([(mn * L + lp, ml, (dn * L + lp) * n, a.offset + (ml * N + dn) * n, n, -1)
                                  for lp in range(L) for dn in range(N)], None, 'in', logical=0))
            # phase 1: a[sl][dn] (filled by local peer sl: flag sl) -> rank (dn, ml), b[sn = mn][sl]
            phases.append(_Phase([(dn * L + ml, mn, (sl * N + dn) * n, b.offset + (mn * L + sl) * n, n, sl)
                                  for dn in range(N) for sl in range(L)], list(range(L)), 'a', 0, logical=1))
            # copy-out of b[sn][sl], filled by rank (sn, ml): flag sn
            phases.append(_Phase([(-1, -1, s * n, s * n, n, s // L) for s in range(W)], list(range(N)), 'b', 1))
            arrivals = {0: N, 1: L}
        elif algo == 'hetu':
            b, c = bufs['b'], bufs['c']
            leader = mn * L
            # phase 0: whole buffer to my leader: a[sl][d]
            phases.append(_Phase([(leader, ml, d * n, a.offset + (ml * W + d) * n, n, -1) for d in range(W)], None, 'in',
                                 logical=0))
            if ml == 0:
                # phase 1 (leaders): a[sl][dn][dl] -> leader of dn, b[sn = mn][dl][sl]
                phases.append(_Phase([(dn * L, mn, (sl * W + dn * L + dl) * n,
                                       b.offset + ((mn * L + dl) * L + sl) * n, n, sl)
                                      for dn in range(N) for dl in range(L) for sl in range(L)],
                                     list(range(L)), 'a', 0, logical=1))
                # phase 2 (leaders): b[sn][dl][sl] -> local rank dl, c[sn][sl]
                phases.append(_Phase([(leader + dl, 0, ((sn * L + dl) * L + sl) * n, c.offset + (sn * L + sl) * n, n, sn)
                                      for dl in range(L) for sn in range(N) for sl in range(L)],
                                     list(range(N)), 'b', 1, logical=2))
            phases.append(_Phase([(-1, -1, s * n, s * n, n, 0) for s in range(W)], [0], 'c', 2))
            arrivals = {0: W, 1: L * L, 2: N * L}
        else:
            raise ValueError('unknown all-to-all algorithm: %s' % algo)
        return phases, arrivals

    def _tables(self, algo, parity, n, bufs):
        key = (algo, parity, n)
        if key not in self.tables:
            phases, arrivals = self._plan(algo, parity, n, bufs)
            dev = self.tr.device
            built = []
            for ph in phases:
                msgs = torch.tensor(ph.msgs, dtype=torch.int64, device=dev).view(-1, 6)
                wait = torch.tensor(ph.wait_idx, dtype=torch.int32, device=dev) if ph.wait_idx else None
                built.append((ph, msgs, wait))
            self.tables[key] = (built, arrivals)
        return self.tables[key]

    # -- run ---------------------------------------------------------------------------------------
    def _ctas(self, algo, logical, n):
        """CTAs per message of a pushing phase.  A function of global quantities only, so that
        every rank (including ranks that do not execute the phase) agrees on the arrival counts."""
        W, L = self.W, self.L
        N = W // L
        count = {'flat': [W], 'pipe': [W], 'dd': [W, W], 'hetu': [W, N * L * L, N * L * L]}[algo][logical]
        return max(1, min(592 // max(count, 1), max(1, n >> 16)))

    def run(self, t, algo='flat', var_len=None, heap_out=False):
        lib = native.lib()
        tr = self.tr
        W = self.W
        t = t.contiguous()
        total = t.numel() * t.element_size()
        assert total % W == 0, "all-to-all payload must split evenly over the ranks"
        n = total // W
        assert n % 16 == 0 and t.data_ptr() % 16 == 0, "per-peer payload must be a multiple of 16 bytes"
        if algo == 'dd' and (self.L == W or self.L == 1):
            algo = 'flat'
        parity = self.calls & 1
        self.calls += 1
        bufs = self._ensure(algo, parity, n)
        built, arrivals = self._tables(algo, parity, n, bufs)
        out = None if heap_out else torch.empty_like(t)
        len_off, len_base = (-1, 0) if var_len is None else (int(var_len[0]), int(var_len[1]))
        result = out

        # cumulative arrivals every flag of every pushing phase will have reached after this call
        for logical, per_call in arrivals.items():
            key = (algo, parity, logical)
            self.arrived[key] = self.arrived.get(key, 0) + per_call * self._ctas(algo, logical, n)

        cur = torch.cuda.current_stream(tr.device)
        budget, status = tr.budget_ms, tr.status_ptr
        bases = bufs['a'].bases_ptr
        side_events = []
        for ph, msgs, wait in built:
            src_ptr = t.data_ptr() if ph.src == 'in' else bufs[ph.src].local_ptr
            want, wait_ptr = 0, 0
            if ph.wait_phase is not None:
                want = self.arrived[(algo, parity, ph.wait_phase)]
                wait_ptr = self._flag_ptr(algo, parity, ph.wait_phase)
            if ph.logical is None:
                ctas = max(1, min(592 // max(msgs.size(0), 1), max(1, n >> 16)))
                flag_off = 0
            else:
                ctas = self._ctas(algo, ph.logical, n)
                flag_off = self._flag_off(algo, parity, ph.logical)
            if ph.stream == 0:
                for ev in side_events:
                    cur.wait_event(ev)
                side_events = []
                if ph.logical is None and heap_out:
                    # last phase without the copy-out: a stream-ordered "everything has arrived" point
                    idx = ph.wait_idx
                    assert idx == list(range(len(idx)))
                    lib.wait_flags(wait_ptr, len(idx), want, budget, status)
                    result = bufs[ph.src].tensor(t.dtype, tuple(t.shape))
                else:
                    lib.xfer(src_ptr, msgs, ctas, bases, flag_off, wait_ptr, wait, want, budget, status,
                             out.data_ptr() if out is not None else 0, len_off, len_base)
            else:
                if self.side is None:
                    self.side = [torch.cuda.Stream(device=tr.device) for _ in range(2)]
                s = self.side[ph.stream - 1]
                s.wait_stream(cur)
                with torch.cuda.stream(s):
                    lib.xfer(src_ptr, msgs, ctas, bases, flag_off, wait_ptr, wait, want, budget, status,
                             out.data_ptr() if out is not None else 0, len_off, len_base)
                    side_events.append(s.record_event())
                t.record_stream(s)
        return result
