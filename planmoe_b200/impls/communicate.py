"""Process groups, plain collectives and autograd-aware collectives (the ``net`` API).

Covers the reference's ``PlanMoE/impls/communicate.py``: world helpers (:18-35), group
construction with OpenMPI/torchrun rendezvous (:42-141), ``simple_*`` collectives
(:148-207), ``AllToAllStatus`` (:210-240), the ``Prim*`` autograd collectives (:385-601)
and the expert permutes (:604-623).

Differences by design: the data plane of the MoE layer is not a private NCCL communicator
but the symmetric-heap transport in ``planmoe_b200.parallel.transport``;
``AllToAllStatus.init`` brings that transport up.  A world of one rank (or no process group
at all) is a first-class case here: every collective degenerates to the identity.
"""

import os
import logging

import torch
import torch.distributed as dist


def _dist_ready():
    return dist.is_available() and dist.is_initialized()


def get_world_size(group=None):
    if not _dist_ready():
        return 1
    try:
        return dist.get_world_size(group)
    except Exception:
        return 1


def get_world_rank(group=None):
    if not _dist_ready():
        return 0
    try:
        return dist.get_rank(group)
    except Exception:
        return 0


def barrier(group=None):
    if get_world_size(group) > 1:
        dist.barrier(group=group)


TUTEL_SKIP_A2A = int(os.environ.get('SKIP_A2A', 0)) > 0


class ParallelPropStorage:
    """Result record of ``create_groups_from_world`` (same attribute names as the reference)."""

    def __repr__(self):
        return ("ParallelPropStorage(global=%d/%d, data_rank=%d of %d groups, model=%d/%d)" % (
            self.global_rank, self.global_size, self.data_rank, self.group_count,
            self.model_rank, self.model_size))


def grid_of(world, rank, group_count):
    """Pure arithmetic of the (data, model) grid: ranks are laid out row-major as ``[group_count][model_size]``.

    Returns ``(group_count, model_size, data_rank, model_rank, rows, cols)`` where ``rows[d]`` lists the ranks of
    model group ``d`` (contiguous) and ``cols[m]`` those of data group ``m`` (strided).  A negative ``group_count``
    asks for model groups of ``-group_count`` ranks.
    """
    if group_count < 0:
        group_count = world // -group_count
    assert group_count > 0 and world % group_count == 0, \
        "Expected to evenly divide devices into %d groups, while the world size of current " \
        "session is %d." % (group_count, world)
    model_size = world // group_count
    rows = [list(range(d * model_size, (d + 1) * model_size)) for d in range(group_count)]
    cols = [list(range(m, world, model_size)) for m in range(model_size)]
    data_rank, model_rank = divmod(rank, model_size)
    return group_count, model_size, data_rank, model_rank, rows, cols


class _World:
    """What this process knows about the job: the one backend it was told to use, its place in the launch
    (torchrun or OpenMPI variables) and every grid it has already built."""

    def __init__(self):
        self.backend = None
        self.grids = {}

    def fix_backend(self, asked):
        if asked:
            if self.backend is None:
                self.backend = asked
            assert self.backend == asked, \
                "Only 1 backend type is allowed, get: %s v.s. %s" % (self.backend, asked)
        return self.backend

    @staticmethod
    def launch_slot():
        """(rank, world, local_rank) as the launcher exported them, or None outside a launcher."""
        env = os.environ
        if 'LOCAL_RANK' in env:
            return int(env.get('RANK', 0)), int(env.get('WORLD_SIZE', 1)), int(env['LOCAL_RANK'])
        if 'OMPI_COMM_WORLD_SIZE' in env:
            return (int(env['OMPI_COMM_WORLD_RANK']), int(env['OMPI_COMM_WORLD_SIZE']),
                    int(env.get('OMPI_COMM_WORLD_LOCAL_RANK', 0)))
        return None

    def connect(self, backend):
        """Bring the default process group up when asked to and not up yet; tell whether one exists."""
        if _dist_ready() or not backend:
            return _dist_ready()
        env, slot = os.environ, self.launch_slot()
        try:
            if slot is not None and 'LOCAL_RANK' not in env:          # OpenMPI: no env:// variables exported
                dist.init_process_group(
                    backend=backend, rank=slot[0], world_size=slot[1],
                    init_method='tcp://%s:%s' % (env['MASTER_ADDR'], env.get('MASTER_PORT', '23456')))
            else:
                dist.init_process_group(backend=backend)
        except ValueError:                                            # env:// without its variables: a lone process
            return False
        return True

    def device_for(self, backend, local_rank):
        if backend is None:
            return None
        if backend == 'gloo':
            return torch.device('cpu')
        if backend == 'nccl':
            dev = torch.device('cuda', min(local_rank, max(torch.cuda.device_count(), 1) - 1))
            if torch.cuda.is_available():
                torch.cuda.set_device(dev)
            return dev
        raise Exception('Unsupported backend type: %s' % backend)


_WORLD = _World()


def _pick_group(memberships, mine, whole_world):
    """Every rank must call ``new_group`` for every membership list, in the same order; keep the one that
    contains this rank.  A single list covering the world is the default group itself."""
    if len(memberships) == 1:
        return whole_world
    made = [dist.new_group(ranks=r) for r in memberships]
    return made[mine]


def create_groups_from_world(group_count, include_init=None):
    """Split the world into ``group_count`` contiguous model groups and the matching strided
    data groups.  ``group_count < 0`` means "groups of size -group_count".

    ``include_init`` names the backend ('nccl' | 'gloo') and also initialises the default
    process group when it is not up yet.  Results are cached per requested ``group_count``.
    """
    backend = _WORLD.fix_backend(include_init)
    if group_count in _WORLD.grids:
        return _WORLD.grids[group_count]

    live = _WORLD.connect(include_init)
    slot = _WORLD.launch_slot()
    world, rank = (dist.get_world_size(), dist.get_rank()) if live else (1, 0)
    local_rank = slot[2] if (live and slot is not None) else 0
    groups, model_size, data_rank, model_rank, rows, cols = grid_of(world, rank, group_count)

    res = ParallelPropStorage()
    res.is_distributed = live
    res.global_size, res.global_rank = world, rank
    res.group_count, res.data_rank = groups, data_rank
    res.model_size, res.model_rank = model_size, model_rank
    res.local_device = _WORLD.device_for(backend, local_rank)
    whole = dist.group.WORLD if live else None
    res.global_group = whole
    res.model_group = _pick_group(rows, data_rank, whole) if live else None
    res.data_group = _pick_group(cols, model_rank, whole) if live else None
    res.dist_print = print if rank == 0 else (lambda *a, **k: None)
    _WORLD.grids[group_count] = res
    return res


def swap_axis(t, x, y):
    return t if x == y else t.swapaxes(x, y)


# ---------------------------------------------------------------------------------------
# Collectives without autograd
# ---------------------------------------------------------------------------------------

def simple_all_reduce(input, group=None, op=dist.ReduceOp.SUM):
    if get_world_size(group) == 1:
        return input
    output = torch.clone(input, memory_format=torch.contiguous_format)
    dist.all_reduce(output, op=op, group=group)
    return output


def simple_all_to_all(input, group=None, background=False):
    world_size = get_world_size(group)
    input = input.contiguous()
    if world_size == 1 or TUTEL_SKIP_A2A:
        return input if not background else (input, lambda *args: None)
    simple_all_to_all._use_builtins = True
    output = torch.empty_like(input)
    if background:
        work = dist.all_to_all_single(output, input, group=group, async_op=True)
        return output, work.wait
    dist.all_to_all_single(output, input, group=group)
    return output


def simple_split(input, group=None):
    world_size = get_world_size(group)
    if world_size == 1:
        return input
    assert input.size(0) % world_size == 0, \
        "Cannot evenly devide dim length %s into %s slices" % (input.size(0), world_size)
    return input.contiguous().chunk(world_size, dim=0)[get_world_rank(group)]


def simple_reduce_scatter(input, group=None, op=dist.ReduceOp.SUM):
    world_size = get_world_size(group)
    if world_size == 1:
        return input
    input = input.contiguous()
    assert input.size(0) % world_size == 0, \
        "Cannot evenly devide dim length %s into %s slices" % (input.size(0), world_size)
    if not input.is_cuda:  # Gloo has no reduce_scatter
        return simple_split(simple_all_reduce(input, group, op=op), group=group)
    output = torch.empty_like(input.chunk(world_size, dim=0)[0])
    dist.reduce_scatter_tensor(output, input, op=op, group=group)
    return output


def simple_all_gather(input, group=None):
    world_size = get_world_size(group)
    if world_size == 1:
        return input
    input = input.contiguous()
    output = torch.empty([world_size * input.size(0)] + list(input.shape[1:]),
                         device=input.device, dtype=input.dtype)
    dist.all_gather_into_tensor(output, input, group=group)
    return output


# ---------------------------------------------------------------------------------------
# Data-plane bootstrap
# ---------------------------------------------------------------------------------------

class AllToAllStatus:
    """Book-keeping for the chunked MoE all-to-all (reference: communicate.py:210-240).

    ``init`` brings up the symmetric-heap transport for ``group`` the first time it is
    called on a CUDA world of more than one rank; CPU worlds and single-rank worlds need
    no set-up (their transport is Gloo all-to-all or the identity).
    """
    initialized = False
    num_split = 0
    split_dim = 0
    max_num_split = 32

    @staticmethod
    def init(group, num_split, split_dim):
        AllToAllStatus.num_split = num_split
        AllToAllStatus.split_dim = split_dim
        if get_world_size(group) <= 1:
            return
        if not AllToAllStatus.initialized:
            if torch.cuda.is_available() and dist.get_backend(group) == 'nccl':
                from ..parallel import transport
                transport.get_transport(group)
            AllToAllStatus.initialized = True


# ---------------------------------------------------------------------------------------
# Collectives with autograd
# ---------------------------------------------------------------------------------------

class RestoreBackward(torch.autograd.Function):
    """Identity on ``input`` whose backward all-to-alls the gradient for ``output``'s producer."""
    @staticmethod
    def forward(ctx, input, output, group=None):
        ctx.group = group
        return input

    @staticmethod
    def backward(ctx, grad_output):
        return (None, simple_all_to_all(grad_output, group=ctx.group), None)


# ---------------------------------------------------------------------------------------
# Stream hand-over and chunked asynchronous all-to-all (autograd Functions)
# ---------------------------------------------------------------------------------------
# The reference declares these Functions on top of native entry points that its extension does not
# bind (communicate.py:243-370; the four stream calls it does bind return their input unchanged,
# custom_kernel.cpp:178-192).  Here they work: a per-device communication stream, one event per
# hand-over index, chunked exchanges that run on that stream and are joined on use.

class _CommStreams:
    streams, events = {}, {}

    @classmethod
    def stream(cls, device):
        key = (device.type, device.index)
        if key not in cls.streams:
            cls.streams[key] = torch.cuda.Stream(device=device)
        return cls.streams[key]

    @classmethod
    def event(cls, device, idx):
        key = (device.type, device.index, int(idx))
        if key not in cls.events:
            cls.events[key] = torch.cuda.Event()
        return cls.events[key]


def _hand_over(t, idx, to_comm):
    """Order the two streams through event ``idx``: work that follows on the receiving stream sees
    everything queued so far on the releasing one.  CPU tensors pass through."""
    if not t.is_cuda:
        return t
    comm, cur = _CommStreams.stream(t.device), torch.cuda.current_stream(t.device)
    ev = _CommStreams.event(t.device, idx)
    src, dst = (cur, comm) if to_comm else (comm, cur)
    ev.record(src)
    dst.wait_event(ev)
    t.record_stream(dst)
    return t


class CurrentStreamRelease(torch.autograd.Function):
    """The compute stream hands ``input`` to the communication stream (backward: takes the gradient back)."""
    @staticmethod
    def forward(ctx, input, idx):
        ctx.idx = idx
        return _hand_over(input.contiguous(), idx, True)

    @staticmethod
    def backward(ctx, grad_output):
        return _hand_over(grad_output, ctx.idx, False), None


class CurrentStreamAcquire(torch.autograd.Function):
    """The compute stream waits for what the communication stream produced under index ``idx``."""
    @staticmethod
    def forward(ctx, input, idx):
        ctx.idx = idx
        return _hand_over(input, idx, False)

    @staticmethod
    def backward(ctx, grad_output):
        return _hand_over(grad_output.contiguous(), ctx.idx, True), None


class NcclStreamRelease(torch.autograd.Function):
    """The communication stream publishes ``input`` under index ``idx`` (the compute stream may acquire it)."""
    @staticmethod
    def forward(ctx, input, idx):
        ctx.idx = idx
        return _hand_over(input, idx, False)

    @staticmethod
    def backward(ctx, grad_output):
        return _hand_over(grad_output, ctx.idx, True), None


class NcclStreamAcquire(torch.autograd.Function):
    """The communication stream waits for what the compute stream released under index ``idx``."""
    @staticmethod
    def forward(ctx, input, idx):
        ctx.idx = idx
        return _hand_over(input, idx, True)

    @staticmethod
    def backward(ctx, grad_output):
        return _hand_over(grad_output, ctx.idx, False), None


def _a2a_chunks(chunks, group, is_compress):
    """All-to-all every chunk (dim 0 split over the ranks); CUDA chunks run back to back on the
    communication stream and the caller's stream joins at the end.  ``is_compress``: ZFP fixed-rate
    8 bits per value around each exchange, as the reference's *_zfp_async entry points intend."""
    if get_world_size(group) == 1:
        return [c.contiguous() for c in chunks]
    codec = None
    if is_compress:
        from ..parallel import codecs
        codec = codecs.get_compressor('zfp')
    world = get_world_size(group)

    def one(c):
        if codec is None:
            return simple_all_to_all(c, group=group)
        packed = codec.compress(c.contiguous(), world)
        wires = [simple_all_to_all(w.view(world, -1), group=group).view(w.shape) for w in packed.wires]
        return codec.decompress(type(packed)(wires, packed.meta))

    if not chunks[0].is_cuda:
        return [one(c) for c in chunks]
    dev = chunks[0].device
    comm, cur = _CommStreams.stream(dev), torch.cuda.current_stream(dev)
    comm.wait_stream(cur)
    with torch.cuda.stream(comm):
        outs = [one(c) for c in chunks]
    cur.wait_stream(comm)
    for t in list(chunks) + outs:
        t.record_stream(comm)
    return outs


def _a2a_two_level(t, group):
    """Equal-split all-to-all along dim 0 through the two-level (2DH) algorithm: on a CUDA world the
    symmetric-heap 'dd' exchange (inside LOCAL_SIZE groups, then between them); elsewhere the flat
    exchange, which delivers the same result."""
    if get_world_size(group) == 1:
        return t
    t = t.contiguous()
    if t.is_cuda and dist.get_backend(group) == 'nccl':
        from ..parallel import transport
        return transport.get_transport(group).all_to_all(t, 'dd')
    return simple_all_to_all(t, group)


class AllToAll2DAsync(torch.autograd.Function):
    """Two-level all-to-all of ``input`` along dim 0; its own adjoint."""
    @staticmethod
    def forward(ctx, input, group=None):
        ctx.group = group
        return _a2a_two_level(input, group)

    @staticmethod
    def backward(ctx, grad_output):
        return _a2a_two_level(grad_output, ctx.group), None


class AllToAllScatterAsync(torch.autograd.Function):
    """Split ``input`` into ``AllToAllStatus.num_split`` chunks along ``AllToAllStatus.split_dim`` and
    all-to-all each chunk; returns the tuple of exchanged chunks.  Backward gathers."""
    @staticmethod
    def forward(ctx, input, is_compress=False, group=None):
        ctx.group, ctx.is_compress = group, bool(is_compress)
        ctx.num_split, ctx.split_dim = max(int(AllToAllStatus.num_split), 1), int(AllToAllStatus.split_dim)
        chunks = [c.contiguous() for c in input.chunk(ctx.num_split, dim=ctx.split_dim)]
        return tuple(_a2a_chunks(chunks, group, ctx.is_compress))

    @staticmethod
    def backward(ctx, *grads):
        outs = _a2a_chunks([g.contiguous() for g in grads], ctx.group, ctx.is_compress)
        return torch.cat(outs, dim=ctx.split_dim), None, None


class AllToAllGatherAsync(torch.autograd.Function):
    """All-to-all each chunk and concatenate them along ``AllToAllStatus.split_dim``.  Backward scatters."""
    @staticmethod
    def forward(ctx, is_compress, *inputs):
        group = None
        ctx.group, ctx.is_compress = group, bool(is_compress)
        ctx.num_split, ctx.split_dim = len(inputs), int(AllToAllStatus.split_dim)
        outs = _a2a_chunks([t.contiguous() for t in inputs], group, ctx.is_compress)
        return torch.cat(outs, dim=ctx.split_dim)

    @staticmethod
    def backward(ctx, grad_output):
        chunks = [c.contiguous() for c in grad_output.chunk(ctx.num_split, dim=ctx.split_dim)]
        return (None,) + tuple(_a2a_chunks(chunks, ctx.group, ctx.is_compress))


def _local_size():
    return int(os.environ.get('LOCAL_SIZE', 1))


class PrimAllToAll2D(torch.autograd.Function):
    """Two-phase hierarchical all-to-all over (data_group, model_group) of LOCAL_SIZE."""
    LOCAL_SIZE = 0

    @staticmethod
    def forward(ctx, x, input_dim, output_dim):
        if PrimAllToAll2D.LOCAL_SIZE == 0:
            PrimAllToAll2D.LOCAL_SIZE = _local_size()
            if PrimAllToAll2D.LOCAL_SIZE == 1:
                logging.warning("LOCAL_SIZE (> 1) for AllToAll 2DH is not set; "
                                "set LOCAL_SIZE or launch through planmoe.launcher.run")
        ctx.input_dim, ctx.output_dim = input_dim, output_dim
        groups = create_groups_from_world(-PrimAllToAll2D.LOCAL_SIZE)
        y = all_to_all(x, input_dim, output_dim, group=groups.data_group)
        y = all_to_all(y, input_dim, output_dim, group=groups.model_group)
        ms, ds = get_world_size(groups.model_group), get_world_size(groups.data_group)
        shape = y.shape
        y = y.view(list(shape[:input_dim]) + [ms, ds, -1] + list(shape[input_dim + 1:]))
        return y.swapaxes(input_dim, input_dim + 1).contiguous().view(shape)

    @staticmethod
    def backward(ctx, dy):
        return (PrimAllToAll2D.apply(dy, ctx.output_dim, ctx.input_dim), None, None)


class PrimAllToAll(torch.autograd.Function):
    @staticmethod
    def forward(ctx, input, group=None):
        ctx.group = group
        return simple_all_to_all(input, group)

    @staticmethod
    def backward(ctx, grad_output):
        return (PrimAllToAll.apply(grad_output, ctx.group), None)

    @staticmethod
    def single(input, group=None):
        return PrimAllToAll.apply(input, group)

    @staticmethod
    def transform(input, input_dim, output_dim, group=None, background=False, use_2dh=False):
        """Generic dim-to-dim all-to-all: gathers ``input_dim`` (it grows W-fold) while
        scattering ``output_dim`` (it shrinks W-fold).  With ``background=True`` returns a
        closure that waits for the transfer and yields the result."""
        if use_2dh:
            assert not background, "Background mode for AllToAll 2DH is not implemented."
            return PrimAllToAll2D.apply(input, input_dim, output_dim)

        world_size = get_world_size(group)
        if input_dim == output_dim or world_size == 1:
            return (lambda *a: input) if background else input

        if input_dim != 0 and output_dim != 0:
            assert not background, 'Unhandle async branch case for flexible all_to_all()'
            t = swap_axis(input, 0, output_dim)
            t = PrimAllToAll.transform(t, input_dim, 0, group)
            return swap_axis(t, 0, output_dim).contiguous()

        if input_dim == 0:
            # scatter output_dim: bring its W-split to the front, exchange, fold into dim 0
            shp = list(input.shape)
            t = input.view(shp[:output_dim] + [world_size, -1] + shp[output_dim + 1:])
            t = t.permute([output_dim] + list(range(output_dim)) +
                          list(range(output_dim + 1, t.dim())))
            out, wait = simple_all_to_all(t, group, background=True)

            def finish():
                wait()
                r = RestoreBackward.apply(out, t, group)
                return r.view([-1] + list(r.shape[2:]))
        else:
            # output_dim == 0: scatter dim 0, received slices are concatenated on input_dim
            t = input
            out, wait = simple_all_to_all(t, group, background=True)

            def finish():
                wait()
                r = RestoreBackward.apply(out, t, group)
                r = r.view([world_size, -1] + list(r.shape[1:]))
                r = r.permute(list(range(1, input_dim + 1)) + [0] +
                              list(range(input_dim + 1, r.dim())))
                return r.contiguous().view(
                    list(r.shape[:input_dim]) + [-1] + list(r.shape[input_dim + 2:]))
        return finish if background else finish()


class PrimBwdAllreduce(torch.autograd.Function):
    """Identity forward, all-reduce of the gradient in backward."""
    @staticmethod
    def forward(ctx, input, op=dist.ReduceOp.SUM, group=None):
        ctx.group, ctx.op = group, op
        return input

    @staticmethod
    def backward(ctx, doutput):
        return (simple_all_reduce(doutput, group=ctx.group, op=ctx.op), None, None)

    @staticmethod
    def transform(input, op=dist.ReduceOp.SUM, group=None):
        return PrimBwdAllreduce.apply(input, op, group)


class PrimFwdAllreduce(torch.autograd.Function):
    """All-reduce forward, identity backward."""
    @staticmethod
    def forward(ctx, input, op=dist.ReduceOp.SUM, group=None):
        return simple_all_reduce(input, group=group, op=op)

    @staticmethod
    def backward(ctx, doutput):
        return (doutput, None, None)

    @staticmethod
    def transform(input, op=dist.ReduceOp.SUM, group=None):
        return PrimFwdAllreduce.apply(input, op, group)


class PrimReducescatter(torch.autograd.Function):
    @staticmethod
    def forward(ctx, input, op=dist.ReduceOp.SUM, group=None):
        ctx.group = group
        return simple_reduce_scatter(input, group, op=op)

    @staticmethod
    def backward(ctx, doutput):
        return (simple_all_gather(doutput, ctx.group), None, None)

    @staticmethod
    def transform(input, dim, group=None):
        t = swap_axis(input, 0, dim)
        t = PrimReducescatter.apply(t, dist.ReduceOp.SUM, group)
        return swap_axis(t, 0, dim)


class PrimAllgather(torch.autograd.Function):
    @staticmethod
    def forward(ctx, input, fused=False, group=None):
        ctx.group, ctx.fused = group, fused
        return simple_all_gather(input, group)

    @staticmethod
    def backward(ctx, doutput):
        if ctx.fused:
            return (simple_reduce_scatter(doutput, ctx.group), None, None)
        return (simple_split(doutput, ctx.group), None, None)

    @staticmethod
    def transform(input, dim, group=None):
        t = swap_axis(input, 0, dim)
        t = PrimAllgather.apply(t, False, group)
        return swap_axis(t, 0, dim)

    @staticmethod
    def zero_gather(input, full_shape=None, group=None):
        """Gather a ZeRO-sharded flat parameter and cut it back to ``full_shape``."""
        if not full_shape:
            full_shape = list(input.shape)
            full_shape[0] *= get_world_size(group)
        numel = 1
        for x in full_shape:
            numel *= int(x)
        gathered = PrimAllgather.apply(input, True, group)
        return gathered.reshape(-1)[:numel].view(list(full_shape))

    @staticmethod
    def zero_scatter(input, scatter_fn, group=None):
        """Flatten + zero-pad to a multiple of the group size, then ``scatter_fn`` it."""
        group_size = get_world_size(group)
        full = input.numel()
        flat = input.reshape(-1)
        if full % group_size != 0:
            padded = torch.zeros([(full + group_size - 1) // group_size * group_size],
                                 device=input.device, dtype=input.dtype)
            padded[:full] = flat
            flat = padded
        return scatter_fn(flat, group=group), input.shape


class PrimSpatialSplit(torch.autograd.Function):
    @staticmethod
    def forward(ctx, input, group=None):
        ctx.group = group
        return simple_split(input, ctx.group)

    @staticmethod
    def backward(ctx, doutput):
        return (simple_all_gather(doutput, ctx.group), None)

    @staticmethod
    def transform(input, dim, group=None):
        t = swap_axis(input, 0, dim)
        t = PrimSpatialSplit.apply(t, group)
        return swap_axis(t, 0, dim)


def pre_expert_permute(input, group=None):
    """[W_src * E_local, c, M] (all-to-all output) -> [E_local, W_src * c, M]."""
    world_size = get_world_size(group)
    if world_size == 1:
        return input
    t = input.view([world_size, -1] + list(input.shape[1:]))      # [W, E_l, c, M]
    t = t.transpose(0, 1).contiguous()                            # [E_l, W, c, M]
    return t.view([t.shape[0], -1] + list(t.shape[3:]))


def post_expert_permute(input, group=None):
    """[E_local, W_src * c, M] -> [W_src * E_local, c, M] (all-to-all input)."""
    world_size = get_world_size(group)
    if world_size == 1:
        return input
    t = input.view([input.shape[0], world_size, -1] + list(input.shape[2:]))  # [E_l, W, c, M]
    t = t.transpose(0, 1).contiguous()                                        # [W, E_l, c, M]
    return t.view([-1] + list(t.shape[2:]))


all_to_all = PrimAllToAll.transform
all_to_all_single = PrimAllToAll.single
zero_gather = PrimAllgather.zero_gather
zero_scatter = PrimAllgather.zero_scatter
all_gather = PrimAllgather.transform
spatial_split = PrimSpatialSplit.transform
reduce_scatter = PrimReducescatter.transform
allreduce_forward = PrimFwdAllreduce.transform
allreduce_backward = PrimBwdAllreduce.transform
