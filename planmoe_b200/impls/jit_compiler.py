"""Run-time compilation of user CUDA kernels (``jit.create_cuda_kernel``).

Reference: ``PlanMoE/impls/jit_compiler.py:1-53`` on top of the native JIT engine
``PlanMoE/custom/jit.h`` (nvcc/NVRTC -> cuModuleLoad -> cuLaunchKernel, launch extents parsed
from ``// [thread_extent] blockIdx.x = N`` comments, kernel name = first ``void`` function).

Here the engine is the native extension's JIT: the source is compiled for ``sm_100a`` by NVRTC
(or, with ``USE_NVRTC=0`` or no libnvrtc, by an ``nvcc --cubin`` child process from the SDK home
set through ``update_sdk_home``), cached per (source, device), and launched on the *current*
stream (the reference launches on the default stream).  ``@key@`` placeholders are substituted
from ``keyword_dict``.
"""

import re

from ..ops import native


def _extents(source):
    dims = {'blockIdx.x': 1, 'blockIdx.y': 1, 'blockIdx.z': 1,
            'threadIdx.x': 1, 'threadIdx.y': 1, 'threadIdx.z': 1}
    for key, val in re.findall(r'//\s*\[thread_extent\]\s*(\w+\.\w)\s*=\s*(\d+)', source):
        if key in dims:
            dims[key] = int(val)
    return dims


def _kernel_name(source):
    m = re.search(r'\bvoid\s+(\w+)\s*\(', source)
    if m is None:
        raise ValueError("no kernel entry (`void name(`) found in source")
    return m.group(1)


class JitCompiler:
    @staticmethod
    def create_raw(source):
        dims = _extents(source)
        name = _kernel_name(source)
        grid = (dims['blockIdx.x'], dims['blockIdx.y'], dims['blockIdx.z'])
        block = (dims['threadIdx.x'], dims['threadIdx.y'], dims['threadIdx.z'])
        state = {}

        def func(*inputs, extra=(), blocks=()):
            import torch
            lib = native.lib()
            if 'fd' not in state:
                state['fd'] = lib.jit_inject_source_raw(source, name)
            g = tuple(blocks) + grid[len(blocks):] if blocks else grid
            with torch.cuda.device(inputs[0].device):
                stream = torch.cuda.current_stream().cuda_stream
                lib.jit_invoke_raw(state['fd'], [int(t.data_ptr()) for t in inputs],
                                   [int(e) for e in extra], list(g), list(block), stream)
        func.compile = lambda: native.lib().jit_compile(
            state.setdefault('fd', native.lib().jit_inject_source_raw(source, name)))
        return func

    @staticmethod
    def generate_kernel(keyword_dict, template):
        for key in keyword_dict:
            template = template.replace('@%s@' % key, str(keyword_dict[key]))
        return JitCompiler.create_raw(template)

    @staticmethod
    def generate_cpu_kernel(kernel_type):
        """CPU scatter (0) / gather (1) / gate-grad (2) loops of the native extension with the
        reference's ``fn(g, i, l, a, b, extra=[samples, dim, capacity])`` convention."""
        from ..jit_kernels import sparse
        return (sparse.create_forward, sparse.create_backward_data,
                sparse.create_backward_gate)[kernel_type](None, False)


def create_cuda_kernel(source, keyword_dict={}):
    return JitCompiler.generate_kernel(keyword_dict, source)
