"""Sparse token <-> expert-slot movement: scatter ("encode"), gather ("decode"), gate-grad.

Three interchangeable backends implement the same three primitives

    scatter(x[S,M], gates[K,S]|None)   -> disp[E*C, M]   disp[idx*C+loc] = g * x      (K1)
    gather (disp[E*C,M], gates|None)   -> out[S, M]      out = sum_k g_k * disp[slot_k] (K2)
    gate_grad(disp[E*C,M], dy[S,M])    -> dg[K, S]       dg_k = <disp[slot_k], dy>      (K3)

* ``cuda``  : hand-written sm_100a kernels (slot-major, atomics-free, bit-reproducible),
* ``cpu``   : the C++ reference loops of the native extension (fp32 / fp64),
* ``torch`` : a composite of differentiable ATen ops (any dtype / device; also the oracle).

They replace the reference's three JIT kernels (``PlanMoE/jit_kernels/sparse.py:17-134``) and
its CPU loops (``PlanMoE/custom/custom_kernel.cpp:57-112``).  A token whose location is
``>= capacity`` (or whose expert id is negative) is dropped: it writes nothing and reads zeros.
"""

import torch

from . import native


class SlotPlan:
    """Stacked routing tensors shared by the three primitives.

    idx, loc : int32 [K, S]   expert id and slot-in-expert of the k-th choice of each token
    E, C     : number of global experts and capacity (slots per expert)
    slot_map : int32 [E*C], value ``t*K+k`` of the (token, choice) that owns the slot, or -1.
               Built lazily; slot ownership is unique, which is what makes the scatter a
               plain store instead of an atomic add.
    """

    def __init__(self, idx, loc, num_experts, capacity, slot_map=None):
        self.idx = idx.contiguous()
        self.loc = loc.contiguous()
        self.K, self.S = int(idx.size(0)), int(idx.size(1))
        self.E, self.C = int(num_experts), int(capacity)
        self._slot_map = slot_map

    @property
    def slot_map(self):
        if self._slot_map is None:
            self._slot_map = build_slot_map(self.idx, self.loc, self.E, self.C)
        return self._slot_map


def build_slot_map(idx, loc, E, C):
    K, S = idx.shape
    if idx.is_cuda:
        return native.lib().build_slot_map(idx, loc, E, C)
    smap = torch.full((E * C,), -1, dtype=torch.int32, device=idx.device)
    tk = (torch.arange(S, device=idx.device, dtype=torch.int32).view(1, S) * K +
          torch.arange(K, device=idx.device, dtype=torch.int32).view(K, 1))
    valid = (loc < C) & (idx >= 0) & (loc >= 0)
    smap[(idx.long() * C + loc.long())[valid]] = tk[valid]
    return smap


# ---------------------------------------------------------------------------------------
# torch composite backend (differentiable by construction)
# ---------------------------------------------------------------------------------------

def scatter_torch(x, plan, gates=None):
    out = x.new_zeros((plan.E * plan.C, x.size(-1)))
    for k in range(plan.K):
        valid = (plan.loc[k] < plan.C) & (plan.idx[k] >= 0)
        slot = (plan.idx[k].long() * plan.C + plan.loc[k].long())[valid]
        src = x[valid]
        if gates is not None:
            src = src * gates[k][valid].unsqueeze(-1).to(x.dtype)
        out = out.index_add(0, slot, src)
    return out


def gather_torch(disp, plan, gates=None):
    out = None
    for k in range(plan.K):
        valid = (plan.loc[k] < plan.C) & (plan.idx[k] >= 0)
        slot = (plan.idx[k].long() * plan.C + plan.loc[k].long()).clamp_(0, plan.E * plan.C - 1)
        rows = disp[slot] * valid.unsqueeze(-1).to(disp.dtype)
        if gates is not None:
            rows = rows * gates[k].unsqueeze(-1).to(disp.dtype)
        out = rows if out is None else out + rows
    return out


def gate_grad_torch(disp, dy, plan):
    res = []
    for k in range(plan.K):
        valid = (plan.loc[k] < plan.C) & (plan.idx[k] >= 0)
        slot = (plan.idx[k].long() * plan.C + plan.loc[k].long()).clamp_(0, plan.E * plan.C - 1)
        res.append((disp[slot].float() * dy.float()).sum(-1) * valid)
    return torch.stack(res)


# ---------------------------------------------------------------------------------------
# native backends
# ---------------------------------------------------------------------------------------

def _native_ok(x):
    if x.is_cuda:
        return x.dtype in (torch.bfloat16, torch.float16, torch.float32)
    return (x.dtype in (torch.float32, torch.float64) and native.available()
            and not native.force_python_fallback())


def _scatter(x, plan, gates):
    x = x.contiguous()
    if x.is_cuda:
        return native.lib().dispatch_scatter(x, plan.slot_map, gates, plan.K, plan.E * plan.C)
    return native.lib().cpu_scatter(x, plan.idx, plan.loc, gates, plan.E, plan.C)


def _gather(disp, plan, gates):
    disp = disp.contiguous()
    if disp.is_cuda:
        return native.lib().dispatch_gather(disp, plan.idx, plan.loc, gates, plan.C)
    return native.lib().cpu_gather(disp, plan.idx, plan.loc, gates, plan.C)


def _gate_grad(disp, dy, plan):
    disp, dy = disp.contiguous(), dy.contiguous()
    if disp.is_cuda:
        return native.lib().dispatch_gate_grad(disp, dy, plan.idx, plan.loc, plan.C)
    return native.lib().cpu_gate_grad(disp, dy, plan.idx, plan.loc, plan.C)


def _gates_for(x, gates):
    """Kernels take gates as fp32 [K,S] on CUDA and in the data dtype on CPU."""
    if gates is None:
        return None
    return gates.detach().to(torch.float32 if x.is_cuda else x.dtype).contiguous()


class _Scatter(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gates, plan):
        ctx.plan = plan
        g = _gates_for(x, gates)
        ctx.save_for_backward(x if gates is not None else None, g)
        ctx.gdtype = gates.dtype if gates is not None else None
        return _scatter(x, plan, g)

    @staticmethod
    def backward(ctx, ddisp):
        x, g = ctx.saved_tensors
        plan = ctx.plan
        ddisp = ddisp.contiguous()
        dx = _gather(ddisp, plan, g)
        dg = None
        if g is not None and ctx.needs_input_grad[1]:
            dg = _gate_grad(ddisp, x, plan).to(ctx.gdtype)
        return dx, dg, None


class _Gather(torch.autograd.Function):
    @staticmethod
    def forward(ctx, disp, gates, plan):
        ctx.plan = plan
        g = _gates_for(disp, gates)
        ctx.save_for_backward(disp if gates is not None else None, g)
        ctx.gdtype = gates.dtype if gates is not None else None
        return _gather(disp, plan, g)

    @staticmethod
    def backward(ctx, dy):
        disp, g = ctx.saved_tensors
        plan = ctx.plan
        dy = dy.contiguous()
        ddisp = _scatter(dy, plan, g)
        dg = None
        if g is not None and ctx.needs_input_grad[1]:
            dg = _gate_grad(disp, dy, plan).to(ctx.gdtype)
        return ddisp, dg, None


def scatter(x, plan, gates=None):
    """Differentiable encode: ``[S, M] -> [E*C, M]`` (w.r.t. ``x`` and ``gates``)."""
    if _native_ok(x):
        return _Scatter.apply(x, gates, plan)
    return scatter_torch(x, plan, gates)


def gather(disp, plan, gates=None):
    """Differentiable decode: ``[E*C, M] -> [S, M]`` (w.r.t. ``disp`` and ``gates``)."""
    if _native_ok(disp):
        return _Gather.apply(disp, gates, plan)
    return gather_torch(disp, plan, gates)
