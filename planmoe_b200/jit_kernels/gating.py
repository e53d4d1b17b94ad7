"""Column-wise ``cumsum - 1`` used to turn one-hot expert masks into slot locations.

Reference: ``PlanMoE/jit_kernels/gating.py:9-22`` (wrapper) and the Blelloch-scan kernel
``PlanMoE/custom/custom_kernel.cpp:331-383``.  Here the CUDA case is one decoupled
block-scan kernel of the native extension (``cumsum_sub_one``); CPU tensors, other ranks or
``FAST_CUMSUM=0`` take ``torch.cumsum - 1``.
"""

import os
import torch

from ..ops import native

use_fast_cumsum = (int(os.environ.get('FAST_CUMSUM', '1')) == 1)


def torch_cumsum_sub_one(mask1):
    return torch.cumsum(mask1, dim=0) - 1


def fast_cumsum_sub_one(data, dim=0):
    if data.dim() != 2 or dim != 0:
        raise Exception("Unimplemented fast_cumsum_sub_one() of data = %s and dim = %s" % (data.size(), dim))
    if not data.is_cuda or not use_fast_cumsum or data.dtype not in (torch.int32, torch.int64):
        return torch_cumsum_sub_one(data)
    out = native.lib().cumsum_sub_one(data.to(torch.int32).contiguous())
    return out.to(data.dtype)


def _tutel_ops_cumsum(x):
    """``torch.ops.tutel_ops.cumsum``: column-wise inclusive cumsum minus one of a 2-D int mask."""
    return fast_cumsum_sub_one(x, dim=0)


def _register_torch_op():
    # The reference exposes its scan kernel as the torch operator tutel_ops::cumsum
    # (PlanMoE/custom/custom_kernel.cpp:385); callers reach it as torch.ops.tutel_ops.cumsum(mask).
    try:
        lib = torch.library.Library('tutel_ops', 'DEF')
        lib.define('cumsum(Tensor x) -> Tensor')
        lib.impl('cumsum', _tutel_ops_cumsum, 'CompositeExplicitAutograd')
        return lib
    except Exception:       # already defined by an earlier import of this module under another name
        return None


_TORCH_LIB = _register_torch_op()
