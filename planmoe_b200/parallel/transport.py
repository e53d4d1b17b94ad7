"""Symmetric-heap transport: the data plane of the MoE layer on CUDA.

One ``Transport`` per process group.  It owns
  * the symmetric heap (``_C.SymmHeap``): a device region per rank, every rank's region mapped
    into every other rank through CUDA IPC, plus a device table of the peers' base addresses;
    buffers are named by byte offset and allocated by a bump allocator that runs in the same
    order on every rank;
  * the status word (``_C.StatusWord``): host-mapped memory where a kernel whose bounded wait
    expired records what it was waiting for; ``check()`` turns that into a Python exception;
  * all-to-all channels (``all_to_all``): flat, Pipe-A2A, HeTu-hierarchical and 2DH exchanges
    built from one generic "wait flags, then copy messages to peers, then signal" kernel.

Synchronisation is by monotonically increasing u64 flags in the destination rank's heap:
a sender's CTA finishes its stores, issues a system-scope fence and a release-add on the flag;
the receiver acquire-polls with a time budget.  Buffers are double-buffered by call parity;
because an all-to-all cannot complete on any rank before every rank has entered it, a rank can
only be two calls ahead of a peer when that peer has finished reading the older buffer.

With a single rank (or in the single-process emulation used by tests) the same kernels run
with the "peer" being the local heap.  The reference's counterpart is the private NCCL
communicator bootstrap and its grouped ncclSend/ncclRecv (``PlanMoE/impls/communicate.py:
210-240``, ``PlanMoE/custom/custom_kernel.cpp:130-176``, ``custom/comm/naive.cpp:11-27``).
"""

import os

import torch
import torch.distributed as dist

from ..ops import native

_ALIGN = 1024
_TRANSPORTS = {}

STATUS_NAMES = {1: 'flag wait timed out', 2: 'mbarrier wait timed out', 3: 'bad argument'}


class TransportError(RuntimeError):
    pass


def default_budget_ms():
    return int(os.environ.get('PLANMOE_WAIT_BUDGET_MS', '20000'))


def debug_guards():
    """PLANMOE_DEBUG_GUARDS=1: every heap block is allocated between two guard bands filled with a canary pattern
    that ``Transport.check()`` verifies, and the fused layer's receive buffers start out filled with NaN so that a
    slot nobody wrote shows up in the output instead of reading as stale zeros.  Stands in for a memory checker."""
    return os.environ.get('PLANMOE_DEBUG_GUARDS', '0') == '1'


_GUARD_BYTES = 1024
_CANARY = 0xA5


class HeapBlock:
    """A block of the symmetric heap: same offset on every rank."""
    __slots__ = ('segment', 'offset', 'nbytes', 'transport')

    def __init__(self, transport, segment, offset, nbytes):
        self.transport, self.segment, self.offset, self.nbytes = transport, segment, offset, nbytes

    @property
    def local_ptr(self):
        return self.transport.segments[self.segment].local_base() + self.offset

    @property
    def bases_ptr(self):
        return self.transport.segments[self.segment].bases_device_ptr()

    @property
    def bases_host(self):
        """Base address of this block's heap segment on every rank, as mapped into this process."""
        seg = self.transport.segments[self.segment]
        return [int(seg.base(r)) for r in range(self.transport.world)]

    def tensor(self, dtype, shape, byte_offset=0):
        """Torch view of this rank's copy of (part of) the block."""
        n = 1
        for s in shape:
            n *= int(s)
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        assert byte_offset + nbytes <= self.nbytes
        raw = native.lib().tensor_from_ptr(self.local_ptr + byte_offset, nbytes, self.transport.device.index)
        return raw.view(dtype).view(*shape)


class Transport:
    def __init__(self, group=None, device=None, emulate=None):
        """``emulate=(rank, world, peers)`` builds one member of a single-process emulation in
        which several logical ranks share one GPU (tests only)."""
        self.group = group
        lib = native.lib()
        if emulate is not None:
            self.rank, self.world = emulate
        elif dist.is_available() and dist.is_initialized():
            self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        else:
            self.rank, self.world = 0, 1
        self.device = torch.device('cuda', torch.cuda.current_device()) if device is None else device
        self.emulated = emulate is not None
        self.segments = []
        self._cursor = []
        self.status = lib.StatusWord()
        self.budget_ms = default_budget_ms()
        self.segment_bytes = int(os.environ.get('PLANMOE_HEAP_MB', '1024')) << 20
        self._a2a = None
        self._peers = None      # emulation: list of sibling transports
        self._guards = []       # (segment, offset of the lower guard, inner bytes) of guarded blocks

    # -- heap -------------------------------------------------------------------------------
    def _new_segment(self, nbytes):
        lib = native.lib()
        seg = lib.SymmHeap(int(nbytes), self.rank, self.world, self.device.index)
        if self.world > 1 and not self.emulated:
            handles = [None] * self.world
            dist.all_gather_object(handles, seg.handle(), group=self.group)
            seg.map_peers(handles)
        self.segments.append(seg)
        self._cursor.append(0)
        return len(self.segments) - 1

    def alloc(self, nbytes):
        """Collective: every rank must call with the same sizes in the same order."""
        if debug_guards():
            inner = (int(nbytes) + _ALIGN - 1) // _ALIGN * _ALIGN
            outer = self._alloc_raw(inner + 2 * _GUARD_BYTES)
            blk = HeapBlock(self, outer.segment, outer.offset + _GUARD_BYTES, inner)
            for off in (outer.offset, outer.offset + _GUARD_BYTES + inner):
                HeapBlock(self, outer.segment, off, _GUARD_BYTES).tensor(torch.uint8, (_GUARD_BYTES,)).fill_(_CANARY)
            self._guards.append((outer.segment, outer.offset, inner))
            return blk
        return self._alloc_raw(nbytes)

    def check_guards(self):
        """Raise if a guard band around any heap block of this rank was overwritten (by any rank)."""
        for seg, off, inner in self._guards:
            for at, name in ((off, 'below'), (off + _GUARD_BYTES + inner, 'above')):
                band = HeapBlock(self, seg, at, _GUARD_BYTES).tensor(torch.uint8, (_GUARD_BYTES,))
                if not bool((band == _CANARY).all()):
                    raise TransportError("rank %d: guard band %s heap block at offset %d (segment %d) was overwritten"
                                         % (self.rank, name, off + _GUARD_BYTES, seg))

    def _alloc_raw(self, nbytes):
        nbytes = (int(nbytes) + _ALIGN - 1) // _ALIGN * _ALIGN
        if self.emulated and self._peers is not None and self is not self._peers[0]:
            raise TransportError("emulated transports allocate through rank 0 (alloc_all)")
        for si in range(len(self.segments)):
            if self._cursor[si] + nbytes <= self.segments[si].size():
                off = self._cursor[si]
                self._cursor[si] += nbytes
                return HeapBlock(self, si, off, nbytes)
        si = self._new_segment(max(nbytes, self.segment_bytes))
        self._cursor[si] = nbytes
        return HeapBlock(self, si, 0, nbytes)

    # -- status -----------------------------------------------------------------------------
    @property
    def status_ptr(self):
        return self.status.device_ptr()

    def check(self, sync=True):
        """Raise if any kernel recorded a failed wait.  ``sync`` first waits for the device."""
        if sync:
            torch.cuda.synchronize(self.device)
        st = self.status.read()
        if st[0] != 0:
            self.status.clear()
            raise TransportError("rank %d: %s (details: %s)" % (
                self.rank, STATUS_NAMES.get(st[0], 'error %d' % st[0]), st[1:4]))
        if self._guards:
            self.check_guards()

    # -- collectives --------------------------------------------------------------------------
    def all_to_all(self, t, algo='flat', var_len=None, heap_out=False):
        """``var_len=(len_off, len_base)``: slices are self-describing and only their valid prefix moves;
        ``heap_out=True``: return a view of the receive buffer in the heap instead of a copy (valid across one
        further call of the same algorithm, see ``parallel/a2a.py``)."""
        from . import a2a
        if self._a2a is None:
            self._a2a = a2a.A2AChannel(self)
        return self._a2a.run(t, algo, var_len=var_len, heap_out=heap_out)

    def close(self):
        for seg in self.segments:
            seg.close()
        self.segments = []


def make_emulated_world(world, device=None):
    """``world`` logical ranks on one GPU in one process.  Their heaps are separate allocations
    and each rank's base table points at the siblings' heaps.  Kernels of different logical ranks
    must never wait on each other across launches (they would not be co-scheduled), so tests
    drive the ranks phase by phase: all pushes of a phase, then all waits."""
    ts = [Transport(emulate=(r, world), device=device) for r in range(world)]
    for t in ts:
        t._peers = ts
    return ts


def emulated_alloc(ts, nbytes):
    """Allocate the same block in every emulated rank and (re)link the base tables."""
    nbytes = (int(nbytes) + _ALIGN - 1) // _ALIGN * _ALIGN
    blocks = []
    for t in ts:
        placed = None
        for si in range(len(t.segments)):
            if t._cursor[si] + nbytes <= t.segments[si].size():
                placed = HeapBlock(t, si, t._cursor[si], nbytes)
                t._cursor[si] += nbytes
                break
        if placed is None:
            lib = native.lib()
            seg = lib.SymmHeap(max(nbytes, t.segment_bytes), t.rank, t.world, t.device.index)
            t.segments.append(seg)
            t._cursor.append(nbytes)
            placed = HeapBlock(t, len(t.segments) - 1, 0, nbytes)
        blocks.append(placed)
    nseg = len(ts[0].segments)
    for si in range(nseg):
        bases = [t.segments[si].local_base() for t in ts]
        for t in ts:
            t.segments[si].map_local(bases)
    return blocks


def get_transport(group=None):
    is_world = group is None or (dist.is_available() and dist.is_initialized() and group is dist.group.WORLD)
    # keyed by the member ranks, not by the object's id (an id can be reused after a group is collected)
    key = 0 if is_world else tuple(dist.get_process_group_ranks(group))
    if key not in _TRANSPORTS:
        _TRANSPORTS[key] = Transport(group)
    return _TRANSPORTS[key]


def reset_transports():
    for t in _TRANSPORTS.values():
        t.close()
    _TRANSPORTS.clear()
