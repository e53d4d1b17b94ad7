"""Chunked pipeline: compress -> all-to-all -> decompress -> experts -> compress -> all-to-all
-> decompress, with ``degree`` chunks in flight.

Reference: ``PlanMoE/impls/overlap.py:12-76`` (autograd triples ``Compress/Comm/Decompress``
around the native FIFO ``compress_operation / comm_operation / decompress_operation`` of
``custom_kernel.cpp:226-288``).

Design differences:
  * Every chunk transfer is an explicit ``ChunkHandle`` object.  The reference pairs the three
    stages of a transfer through global counters indexed by call order, which ties it to 32
    slots and to autograd's replay order; a handle has no such coupling, so any number of MoE
    layers and chunks can be in flight.
  * On CUDA the codec + all-to-all of a chunk are enqueued on a side stream and joined by
    events, so chunk i's transfers overlap chunk i-1's expert GEMMs, in forward and backward.
  * A world of one rank works (identity transport).

This is the generic path (any codec, any comm algorithm, custom experts, CPU).  The bf16 FFN
layer on CUDA takes the fused kernels in ``planmoe_b200.ops.fused_moe`` instead.
"""

import torch

from . import communicate as C
from ..parallel import codecs, comms

_SIDE_STREAMS = {}


def _side_stream(device):
    key = (device.type, device.index)
    if key not in _SIDE_STREAMS:
        _SIDE_STREAMS[key] = torch.cuda.Stream(device=device)
    return _SIDE_STREAMS[key]


class ChunkHandle:
    """One codec + all-to-all transfer of one tensor: ``launch`` then ``finish``."""

    def __init__(self, compress_name, comm_name, group, overlap=True):
        self.codec = codecs.get_compressor(compress_name)
        self.comm = comms.get_comm(comm_name, group)
        self.overlap = overlap
        self.packed = None
        self.event = None

    def _run(self, t):
        packed = self.codec.compress(self.comm.pre_comm(t), self.comm.world_size)
        var_len = getattr(packed, 'var_len', None)
        if var_len is not None and hasattr(self.comm, 'all_to_all_var'):
            packed.wires = [self.comm.all_to_all_var(packed.wires[0], *var_len)] + \
                           [self.comm.all_to_all(w) for w in packed.wires[1:]]
        else:
            packed.wires = [self.comm.all_to_all(w) for w in packed.wires]
        return packed

    def launch(self, t):
        if t.is_cuda and self.overlap and self.comm.world_size > 1:
            cur = torch.cuda.current_stream(t.device)
            side = _side_stream(t.device)
            side.wait_stream(cur)
            with torch.cuda.stream(side):
                self.packed = self._run(t)
                for w in self.packed.wires:
                    w.record_stream(cur)
                self.event = side.record_event()
            t.record_stream(side)
        else:
            self.packed = self._run(t)
        return self

    def finish(self):
        if self.event is not None:
            torch.cuda.current_stream().wait_event(self.event)
        out = self.codec.decompress(self.packed)
        self.packed = None
        return out


class _Link:
    """Joins the launch and finish halves of one transfer (and of its gradient transfer)."""
    __slots__ = ('args', 'fwd', 'bwd')

    def __init__(self, compress_name, comm_name, group):
        self.args = (compress_name, comm_name, group)
        self.fwd = self.bwd = None


class _Launch(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, link):
        ctx.link = link
        link.fwd = ChunkHandle(*link.args).launch(x)
        return x.new_empty(0)            # ordering token consumed by _Finish

    @staticmethod
    def backward(ctx, _token_grad):
        handle, ctx.link.bwd = ctx.link.bwd, None
        return handle.finish(), None


class _Finish(torch.autograd.Function):
    @staticmethod
    def forward(ctx, token, link):
        ctx.link = link
        handle, link.fwd = link.fwd, None
        return handle.finish()

    @staticmethod
    def backward(ctx, grad):
        ctx.link.bwd = ChunkHandle(*ctx.link.args).launch(grad.contiguous())
        return grad.new_empty(0), None


# The reference's stage names, kept as aliases of the two halves.
Compress = _Launch
Decompress = _Finish


def coded_all_to_all_launch(x, compress_name, comm_name, group):
    link = _Link(compress_name, comm_name, group)
    return _Launch.apply(x, link), link


def coded_all_to_all_finish(token, link):
    return _Finish.apply(token, link)


def a2a_ffn_overlap_forward(input, expert_fn, a2a_ffn_overlap_degree, use_2dh, group,
                            compress_name='no', comm_name='naive'):
    """``input`` is ``[E_global, C, M]``; returns the same shape after the experts ran on their
    home ranks.  ``use_2dh=True`` selects the 2DH algorithm when ``comm_name`` is the default."""
    degree = int(a2a_ffn_overlap_degree)
    split_dim = 1
    assert degree <= C.AllToAllStatus.max_num_split, \
        "Excepting a2a_ffn_overlap_degree (%d) <= AllToAllStatus.max_num_split (%d)." % (
            degree, C.AllToAllStatus.max_num_split)
    assert input.shape[split_dim] % degree == 0, \
        "Excepting input.shape[%d] (%d) be multiple of a2a_ffn_overlap_degree (%d)." % (
            split_dim, input.shape[split_dim], degree)
    C.AllToAllStatus.init(group, degree, split_dim)
    if use_2dh and comm_name == 'naive':
        comm_name = 'dd'

    chunks = list(input.split(input.shape[split_dim] // degree, dim=split_dim))
    pending = [coded_all_to_all_launch(c.contiguous(), compress_name, comm_name, group)
               for c in chunks]
    for i in range(degree):
        x = coded_all_to_all_finish(*pending[i])
        y = C.post_expert_permute(expert_fn(C.pre_expert_permute(x, group=group)), group=group)
        pending[i] = coded_all_to_all_launch(y.contiguous(), compress_name, comm_name, group)
    outs = [coded_all_to_all_finish(*p) for p in pending]
    return outs[0] if degree == 1 else torch.cat(outs, dim=split_dim)
