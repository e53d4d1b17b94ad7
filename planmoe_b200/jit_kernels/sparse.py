"""Call-compatible factories for the three dispatch primitives.

The reference builds these at run time from CUDA-C strings through its JIT
(``PlanMoE/jit_kernels/sparse.py:17-134``).  Here they are ahead-of-time sm_100a kernels (and C++
CPU loops); the factories only adapt the reference's calling convention

    fn(gates, indices, locations, a, b, extra=[samples, aligned_dim, capacity])

to ``planmoe_b200.ops.dispatch``.  ``gates`` is one ``[S]`` (or ``[S, 2]`` replicated) tensor for
a single choice k; the functions work in place on their output argument as the originals do.
"""

import torch

from ..ops import dispatch as D


def _gate_column(g, samples, like):
    g = g.reshape(g.size(0), -1)[:samples, 0]
    return g.reshape(1, -1).to(like.dtype)


def _plan(indices, locations, out_rows, capacity):
    idx = indices.reshape(1, -1).to(torch.int32)
    loc = locations.reshape(1, -1).to(torch.int32)
    return D.SlotPlan(idx, loc, out_rows // capacity, capacity)


def create_forward(param_dtype, is_cuda=True):
    """K1: ``dispatched[idx*C+loc] += gate * x`` (slots are unique, so the add is a store
    on top of what the buffer already holds)."""
    def fwd(gates, indices, locations, reshaped_input, dispatched_input, extra=()):
        samples, _, capacity = extra
        plan = _plan(indices, locations, dispatched_input.size(0), capacity)
        upd = D._scatter(reshaped_input, plan, D._gates_for(reshaped_input, _gate_column(gates, samples, reshaped_input)))
        dispatched_input.add_(upd.view_as(dispatched_input))
    return fwd


def create_backward_data(param_dtype, is_cuda=True):
    """K2: ``out[t] = gate[t] * dispatched[idx*C+loc]`` (zero row when dropped)."""
    def bwd_data(gates, indices, locations, grad_reshaped_input, dispatched_input, extra=()):
        samples, _, capacity = extra
        plan = _plan(indices, locations, dispatched_input.size(0), capacity)
        res = D._gather(dispatched_input, plan, D._gates_for(dispatched_input, _gate_column(gates, samples, dispatched_input)))
        grad_reshaped_input.copy_(res.view_as(grad_reshaped_input))
    return bwd_data


def create_backward_gate(param_dtype, is_cuda=True):
    """K3: ``grad_gates[t] = <dispatched[idx*C+loc], x[t]>``."""
    def bwd_gate(grad_gates, indices, locations, reshaped_input, dispatched_input, extra=()):
        samples, _, capacity = extra
        plan = _plan(indices, locations, dispatched_input.size(0), capacity)
        res = D._gate_grad(dispatched_input, reshaped_input, plan)
        grad_gates.reshape(-1)[:samples].copy_(res.reshape(-1).to(grad_gates.dtype))
    return bwd_gate
