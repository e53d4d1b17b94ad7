"""Top-k routing (``extract_critical``) and the encode / decode dispatcher.

API parity with the reference's ``PlanMoE/impls/fast_dispatch.py``: ``extract_critical``
(:140-195) returns ``((E, indices_s, locations_s, gates_s, capacity), l_loss)``;
``fast_encode`` (:197-201) gives ``[E, C, M]``; ``fast_decode`` (:203-207) gives ``[S, M]``;
``TutelMoeFastDispatcher`` (:82-131) keeps its ``update / encode / decode`` methods.

Routing rules kept bit-for-bit (they fix which token lands in which slot):
  * top-k on softmax scores; gate_k = score of the k-th pick,
  * slot location = running count of earlier tokens that picked the same expert, where every
    k-th pick ranks after all (k-1)-th picks of that expert,
  * ``normalize_gate`` divides by the clamped sum over k (only when k > 1),
  * capacity = k * int(cf * ceil(S/E)); cf == 0 -> dynamic (max location + 1, MAX-reduced);
    cf < 0 -> min(dynamic, bound from |cf|); then rounded up to ``alignment``,
  * a pick whose location >= capacity is dropped.

Unlike the reference, bf16 data is moved by a native bf16 kernel (no fp32 round trip) and the
scatter is a unique-slot store instead of an atomic add.
"""

import torch

from . import losses
from .communicate import simple_all_reduce
from ..jit_kernels.gating import fast_cumsum_sub_one
from ..ops import dispatch as D


class RoutingPlan(tuple):
    """The 5-tuple ``(E, indices_s, locations_s, gates_s, capacity)`` plus cached stacked
    tensors for the kernels (``.slots`` is an ``ops.dispatch.SlotPlan``)."""

    def __new__(cls, num_experts, indices_s, locations_s, gates_s, capacity, slots=None):
        self = super().__new__(cls, (num_experts, indices_s, locations_s, gates_s, capacity))
        self._slots = slots
        return self

    @property
    def slots(self):
        if self._slots is None:
            idx = torch.stack([x.to(torch.int32).view(-1) for x in self[1]])
            loc = torch.stack([x.to(torch.int32).view(-1) for x in self[2]])
            self._slots = D.SlotPlan(idx, loc, self[0], self[4])
        return self._slots

    def stacked_gates(self):
        return torch.stack(list(self[3]))


def _as_plan(crit):
    if isinstance(crit, RoutingPlan):
        return crit
    return RoutingPlan(*crit)


def compute_sorted_location(x, importance_scores):
    """Batch-prioritised routing: locations are assigned in order of token importance
    (lowest ``importance_scores`` first) instead of token order."""
    order = importance_scores.argsort(dim=0)
    sorted_x = x[order]
    sorted_loc = fast_cumsum_sub_one(sorted_x) * sorted_x
    out = torch.empty_like(sorted_loc)
    out[order] = sorted_loc
    return out


def extract_critical(scores, top_k, loss_fn=losses.gshard_loss, capacity_factor=1.0,
                     batch_prioritized_routing=False, normalize_gate=True, group=None, alignment=1):
    S, E = int(scores.size(0)), int(scores.size(1))
    top_k = min(int(top_k), E)
    topk_indices = torch.topk(scores, top_k, dim=1).indices
    gates_all = scores.gather(1, topk_indices)                      # [S, k], differentiable

    l_loss = loss_fn(scores, topk_indices) if loss_fn is not None else None

    if batch_prioritized_routing:
        importance = -scores.max(dim=1)[0]
        locate = lambda m: compute_sorted_location(m, importance)   # noqa: E731
    else:
        locate = fast_cumsum_sub_one

    indices_s, locations_s = [], []
    base = None
    for k in range(top_k):
        ids = topk_indices[:, k]
        mask = losses._one_hot_with_dtype(ids, E, dtype=torch.int32)
        pos = locate(mask)
        if base is not None:
            pos = pos + base
        locations_s.append(pos.gather(1, ids.view(-1, 1)).view(-1).to(torch.int32))
        indices_s.append(ids.to(torch.int32))
        counts = mask.sum(dim=0, keepdim=True)
        base = counts if base is None else base + counts

    gates_s = [gates_all[:, k] for k in range(top_k)]
    if top_k > 1 and normalize_gate:
        denom = torch.clamp(gates_all.sum(dim=1), min=torch.finfo(scores.dtype).eps)
        gates_s = [g / denom for g in gates_s]

    per_expert = (S + E - 1) // E
    if capacity_factor > 0:
        capacity = top_k * int(capacity_factor * per_expert)
    else:
        peak = torch.max(torch.cat(locations_s, dim=0))
        capacity = int(simple_all_reduce(peak, group=group, op=torch.distributed.ReduceOp.MAX)) + 1
        if capacity_factor < 0:
            capacity = min(capacity, top_k * int(-capacity_factor * per_expert))
    if capacity % alignment:
        capacity += alignment - capacity % alignment

    return RoutingPlan(E, indices_s, locations_s, gates_s, capacity), l_loss


class TutelMoeFastDispatcher:
    """Stateful encode/decode helper (reference: fast_dispatch.py:82-131)."""

    def __init__(self, num_global_experts, capacity, model_dim, dispatch_dtype):
        self.num_global_experts = int(num_global_experts)
        self.capacity = int(capacity)
        self.model_dim = int(model_dim)
        self.dtype = dispatch_dtype
        self.original_dtype = dispatch_dtype
        self.is_postscore = True
        self._plan = None

    def update(self, indices_, locations_, gates_, capacity=None, is_postscore=True):
        self.capacity = int(capacity) or self.capacity
        self.indices_ = [x.to(torch.int32).view(-1) for x in indices_]
        self.locations_ = [x.to(torch.int32) for x in locations_]
        self.gates_ = list(gates_)
        self.is_postscore = is_postscore
        self.sample_size = int(self.indices_[0].size(0))
        self._plan = RoutingPlan(self.num_global_experts, self.indices_, self.locations_,
                                 self.gates_, self.capacity)

    def _gates(self, like):
        return torch.stack([g.to(like.dtype) for g in self.gates_])

    def encode(self, data):
        gates = None if self.is_postscore else self._gates(data)
        return D.scatter(data, self._plan.slots, gates)

    def decode(self, data):
        gates = self._gates(data) if self.is_postscore else None
        return D.gather(data.reshape(-1, data.size(-1)), self._plan.slots, gates)


fast_dispatcher = TutelMoeFastDispatcher


def fast_encode(data, critial_data, is_postscore=True):
    """[S, M] tokens -> [E, C, M] expert slots (gate-weighted iff ``not is_postscore``)."""
    plan = _as_plan(critial_data)
    gates = None if is_postscore else plan.stacked_gates().to(data.dtype)
    return D.scatter(data, plan.slots, gates).view(plan[0], -1, data.size(-1))


def fast_decode(data, critial_data, is_postscore=True):
    """[E, C, M] expert slots -> [S, M] tokens (gate-weighted iff ``is_postscore``)."""
    plan = _as_plan(critial_data)
    gates = plan.stacked_gates().to(data.dtype) if is_postscore else None
    return D.gather(data.reshape(-1, data.size(-1)), plan.slots, gates)
