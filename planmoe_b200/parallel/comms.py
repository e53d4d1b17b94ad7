"""All-to-all algorithms behind the ``comm_name`` switch of the MoE layer.

Python face of the ``AbstractComm`` extension point (reference:
``PlanMoE/custom/comm/abstract.h:10-24``) and its four algorithms:

  naive  flat exchange, one message per peer                      (``comm/naive.cpp:11-27``)
  pipe   Pipe-A2A: intra-group and inter-group peers progress     (``comm/pipe.cpp:12-31``)
         concurrently on two independent channels
  hetu   hierarchical: gather to group leader, leaders exchange,  (``comm/hetu.cpp:15-76``)
         leader scatters; layout transforms in between
  dd     2DH: intra-group exchange then inter-group exchange      (``dd_comm.cpp:15-90``)
  nccl   torch.distributed ``all_to_all_single`` (the measured baseline transport)

Every algorithm takes a tensor whose dim 0 is split evenly over the W destination ranks and
returns the tensor whose dim 0 is the concatenation over the W source ranks.  "Group" means
``LOCAL_SIZE`` consecutive ranks (env, default: all ranks); on one NVSwitch box
``LOCAL_SIZE=4`` gives the two logical 4-GPU groups.

On CUDA worlds the moves are SM-driven peer stores of the symmetric-heap transport
(``planmoe_b200.parallel.transport``); on CPU (Gloo) worlds the same index arithmetic runs on
``torch.distributed`` primitives, which is what the multi-process CPU tests exercise.
Unknown names fall back to ``naive`` like the reference factory (``custom_kernel.cpp:209-224``).
"""

import os

import torch
import torch.distributed as dist

from ..impls import communicate as C


def local_size(world):
    ls = int(os.environ.get('LOCAL_SIZE', 0)) or world
    ls = min(ls, world)
    return ls if world % ls == 0 else world


class AbstractComm:
    name = 'abstract'

    def __init__(self, group=None):
        self.group = group
        self.world_size = C.get_world_size(group)
        self.world_rank = C.get_world_rank(group)
        self.local_size = local_size(self.world_size)
        self.local_rank = self.world_rank % self.local_size

    # -- extension points ---------------------------------------------------------------
    def pre_comm(self, t):
        return t

    def all_to_all(self, t):
        raise NotImplementedError

    def all_to_all_var(self, t, len_off, len_base):
        """All-to-all of self-describing slices: ``t`` is ``[W, cap]`` bytes and the u32 at byte ``len_off`` of
        every slice holds how many bytes follow its ``len_base`` bytes of header.  Returns ``[W, width]`` with
        ``width <= cap``; bytes past a slice's own length are undefined.

        On the symmetric-heap transport the kernels read the sizes on the device and move only the valid
        prefix of each slice (no host synchronisation, so the call can be captured in a CUDA graph).  The
        library collectives behind the CPU / NCCL transports need one width for all ranks: the ranks agree on
        the maximum with one all-reduce and a host read."""
        t = t.contiguous()
        if self.world_size == 1 or C.TUTEL_SKIP_A2A:
            return t
        algo = getattr(self, 'algo', None)
        if algo is not None and self._use_transport(t):
            return self._transport().all_to_all(t, algo=algo, var_len=(len_off, len_base))
        sizes = t[:, len_off:len_off + 4].contiguous().view(torch.int32).view(-1).to(torch.int64) + len_base
        width = sizes.max().reshape(1)
        dist.all_reduce(width, op=dist.ReduceOp.MAX, group=self.group)
        width = min((int(width.item()) + 15) // 16 * 16, t.size(1))
        return self.all_to_all(t[:, :width].contiguous())

    # -- helpers ------------------------------------------------------------------------
    def _use_transport(self, t):
        return t.is_cuda and self.world_size > 1

    def _transport(self):
        from . import transport
        return transport.get_transport(self.group)


def _gloo_a2a(t, group):
    out = torch.empty_like(t)
    dist.all_to_all_single(out, t, group=group)
    return out


class NaiveComm(AbstractComm):
    name, algo = 'naive', 'flat'

    def all_to_all(self, t):
        if self.world_size == 1 or C.TUTEL_SKIP_A2A:
            return t
        t = t.contiguous()
        if self._use_transport(t):
            return self._transport().all_to_all(t, algo='flat')
        return _gloo_a2a(t, self.group)


class NcclComm(AbstractComm):
    """Baseline: the collective library's own all-to-all."""
    name = 'nccl'

    def all_to_all(self, t):
        if self.world_size == 1 or C.TUTEL_SKIP_A2A:
            return t
        return _gloo_a2a(t.contiguous(), self.group)


class PipeComm(AbstractComm):
    """Pipe-A2A: peers inside my group and peers outside it are served by two independent
    channels that run concurrently."""
    name, algo = 'pipe', 'pipe'

    def all_to_all(self, t):
        if self.world_size == 1 or C.TUTEL_SKIP_A2A:
            return t
        t = t.contiguous()
        if self._use_transport(t):
            return self._transport().all_to_all(t, algo='pipe')
        W, L, me = self.world_size, self.local_size, self.world_rank
        out = torch.empty_like(t)
        src, dst = t.view(W, -1), out.view(W, -1)
        dst[me].copy_(src[me])
        my_group = me // L
        for intra in (True, False):          # two independent batches of point-to-point ops
            ops = []
            for p in range(W):
                if p == me or ((p // L) == my_group) != intra:
                    continue
                gp = dist.get_global_rank(self.group, p) if self.group is not None else p
                ops.append(dist.P2POp(dist.isend, src[p], gp, group=self.group))
                ops.append(dist.P2POp(dist.irecv, dst[p], gp, group=self.group))
            if ops:
                for w in dist.batch_isend_irecv(ops):
                    w.wait()
        return out


def _subgroups(L):
    """(intra-group pg, same-local-rank pg) for groups of L consecutive world ranks."""
    g = C.create_groups_from_world(-L)
    return g.model_group, g.data_group


class DdComm(AbstractComm):
    """2DH: phase 1 exchanges inside the group so that every rank holds what its group sends
    to its own local index everywhere; phase 2 exchanges between groups."""
    name, algo = 'dd', 'dd'

    def all_to_all(self, t):
        W, L = self.world_size, self.local_size
        if W == 1 or C.TUTEL_SKIP_A2A:
            return t
        t = t.contiguous()
        if L == W or L == 1:
            return NaiveComm(self.group).all_to_all(t)
        if self._use_transport(t):
            return self._transport().all_to_all(t, algo='dd')
        assert self.group is None or self.group == dist.group.WORLD, \
            "hierarchical CPU path works on the world group"
        N = W // L
        intra, inter = _subgroups(L)
        x = t.view(N, L, -1).transpose(0, 1).contiguous()        # [dl][dn][n]
        x = _gloo_a2a(x, intra)                                  # [sl][dn][n]
        x = x.view(L, N, -1).transpose(0, 1).contiguous()        # [dn][sl][n]
        x = _gloo_a2a(x, inter)                                  # [sn][sl][n]
        return x.view(t.shape)


class HeTuComm(AbstractComm):
    """Hierarchical leader algorithm: gather -> transform -> leaders' exchange -> transform
    -> scatter.  Works for any dtype and rank of tensor (the reference's scratch sizing only
    fits 2-D fp32)."""
    name, algo = 'hetu', 'hetu'

    def all_to_all(self, t):
        W, L = self.world_size, self.local_size
        if W == 1 or C.TUTEL_SKIP_A2A:
            return t
        t = t.contiguous()
        if L == W and not t.is_cuda:
            pass  # one group: leader gathers everything, transforms, scatters
        if self._use_transport(t):
            return self._transport().all_to_all(t, algo='hetu')
        assert self.group is None or self.group == dist.group.WORLD, \
            "hierarchical CPU path works on the world group"
        N = W // L
        intra, inter = _subgroups(L)
        me = self.world_rank
        leader = (me // L) * L
        is_leader = (me == leader)
        flat = t.view(-1)
        gathered = [torch.empty_like(flat) for _ in range(L)] if is_leader else None
        dist.gather(flat, gathered, dst=leader, group=intra)
        scatter_list = None
        if is_leader:
            x = torch.stack(gathered).view(L, N, L, -1)          # [sl][dn][dl][n]
            x = x.permute(1, 2, 0, 3).contiguous()               # [dn][dl][sl][n]
            if N > 1:
                x = _gloo_a2a(x, inter)                          # [sn][dl][sl][n]
            x = x.view(N, L, L, -1).permute(1, 0, 2, 3).contiguous()   # [dl][sn][sl][n]
            scatter_list = [x[i].reshape(-1) for i in range(L)]
        out = torch.empty_like(flat)
        dist.scatter(out, scatter_list, src=leader, group=intra)
        return out.view(t.shape)


_REGISTRY = {}


def register_comm(name, factory):
    """Register ``factory(group) -> AbstractComm`` under ``name`` (overrides built-ins)."""
    _REGISTRY[name] = factory


class NativeComm(AbstractComm):
    """Bridge to an all-to-all algorithm registered in C++ (``planmoe::register_comm``; extension contract in
    ``csrc/comm/abstract.h``).  The C++ object is kept alive across calls; on CUDA worlds it is given a block of
    the symmetric heap (the same offset on every rank) that it lays out itself, the table of the peers' heap base
    addresses, the status word and the wait budget, which is all a user algorithm needs to move data between
    ranks with ``planmoe::launch_xfer`` or kernels of its own."""

    _HANDLES = {}

    def __init__(self, name, group=None):
        super().__init__(group)
        self.name = name

    def _handle(self, t):
        from ..ops import native
        lib = native.lib()
        nbytes = t.numel() * t.element_size()
        ranks = tuple(dist.get_process_group_ranks(self.group)) if (self.group is not None and self.world_size > 1) else ()
        key = (self.name, ranks, self.world_size, t.is_cuda and self.world_size > 1)
        cur = NativeComm._HANDLES.get(key)
        if cur is not None and cur[1] >= nbytes:
            return cur[0]
        if not (t.is_cuda and self.world_size > 1):
            h = lib.NativeCommHandle(self.name, self.world_size, self.world_rank, self.local_size)
            NativeComm._HANDLES[key] = (h, 1 << 62)
            return h
        tr = self._transport()
        cap = 1 << 20
        while cap < nbytes:
            cap <<= 1
        probe = lib.NativeCommHandle(self.name, self.world_size, self.world_rank, self.local_size)
        blk = tr.alloc(probe.scratch_bytes_for(cap))             # collective: every rank asks for the same size
        h = lib.NativeCommHandle(self.name, self.world_size, self.world_rank, self.local_size, blk.bases_ptr,
                                 tr.segments[blk.segment].local_base(), blk.offset, blk.nbytes, tr.status_ptr,
                                 tr.budget_ms)
        NativeComm._HANDLES[key] = (h, cap)
        return h

    def all_to_all(self, t):
        if C.TUTEL_SKIP_A2A:
            return t
        t = t.contiguous()
        if self.world_size > 1 and not t.is_cuda:
            return _gloo_a2a(t, self.group)                      # CPU worlds have no heap: the library collective
        return self._handle(t).all_to_all(t)


def get_comm(name, group=None):
    factory = _REGISTRY.get(name)
    if factory is None:
        from ..ops import native
        lib = native.maybe_lib()
        if lib is not None and name in lib.native_comm_names():
            return NativeComm(name, group)
        factory = NaiveComm
    return factory(group)


for _cls in (NaiveComm, NcclComm, PipeComm, DdComm, HeTuComm):
    register_comm(_cls.name, _cls)
