"""Reference-named native entry points (module alias: ``schemoe_custom_kernel``).

The reference's extension binds these in ``PlanMoE/custom/custom_kernel.cpp:292-321``.  Scripts
written against it (e.g. ``PlanMoE/examples/pre_test.py:192-210``) call

    compress_operation(x, codec, comm) -> comm_operation(t) -> decompress_operation(t)

and rely on three global counters to pair the calls.  Here the same call sequence is served by a
FIFO of explicit ``ChunkHandle`` objects (no 32-slot event table, so any number of transfers may be
in flight); ``clear_ptr_lst`` empties it.  The NCCL bootstrap functions are kept as harmless shims:
the data plane is the symmetric heap, which ``init_nccl`` brings up.
"""

import torch

from ..impls.overlap import ChunkHandle
from ..ops import native
from ..parallel import codecs as _codecs

_FIFO = []
_COMM_CNT = 0
_DECOMPRESS_CNT = 0


def clear_ptr_lst():
    global _COMM_CNT, _DECOMPRESS_CNT
    _FIFO.clear()
    _COMM_CNT = _DECOMPRESS_CNT = 0


def compress_operation(input, compress_name, comm_name):
    h = ChunkHandle(compress_name, comm_name, None, overlap=False)
    h.packed = h.codec.compress(h.comm.pre_comm(input), h.comm.world_size)
    _FIFO.append(h)
    return h.packed.wires[0]


def comm_operation(input):
    global _COMM_CNT
    h = _FIFO[_COMM_CNT]
    _COMM_CNT += 1
    h.packed.wires = [h.comm.all_to_all(w) for w in h.packed.wires]
    return h.packed.wires[0]


def decompress_operation(input):
    global _DECOMPRESS_CNT
    h = _FIFO[_DECOMPRESS_CNT]
    _DECOMPRESS_CNT += 1
    out = h.codec.decompress(h.packed)
    h.packed = None
    return out


# -- bootstrap shims ----------------------------------------------------------------------------
def get_nccl_unique_id_size():
    return 128


def get_nccl_unique_id(tensor):
    tensor.zero_()
    return tensor


def init_nccl(unique_ids, world_size, world_rank, max_num_split):
    if torch.cuda.is_available() and world_size > 1:
        from ..parallel import transport
        transport.get_transport(None)


def current_stream_release(t, idx=0):
    return t


def current_stream_acquire(t, idx=0):
    return t


def nccl_stream_release(t, idx=0):
    return t


def nccl_stream_acquire(t, idx=0):
    return t


# -- JIT + CPU sparse ops -------------------------------------------------------------------------
def update_sdk_home(path):
    home = bytes(path.tolist()).decode() if isinstance(path, torch.Tensor) else str(path)
    native.lib().update_sdk_home(home)


_SOURCES = []


def inject_source(source):
    from ..impls.jit_compiler import JitCompiler
    _SOURCES.append(JitCompiler.create_raw(source))
    return len(_SOURCES) - 1


def invoke(tensors, extra, blocks, fd):
    _SOURCES[fd](*tensors, extra=extra, blocks=blocks)


def _invoke_cpu(tensors, extra, kernel_type):
    from ..impls.jit_compiler import JitCompiler
    g, i, l, a, b = tensors
    JitCompiler.generate_cpu_kernel(kernel_type)(g, i, l, a, b, extra=extra)


def invoke_cpu_fp32(tensors, extra, kernel_type):
    _invoke_cpu(tensors, extra, kernel_type)


def invoke_cpu_fp64(tensors, extra, kernel_type):
    _invoke_cpu(tensors, extra, kernel_type)


register_compressor = _codecs.register_compressor
