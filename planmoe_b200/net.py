"""Facade: collectives and the ZeRO-style optimizer wrapper (reference ``PlanMoE/net.py:6-56``)."""

from .impls.communicate import get_world_size, get_world_rank, create_groups_from_world, barrier
from .impls.communicate import (simple_all_reduce, simple_all_to_all, simple_split,
                                simple_reduce_scatter, simple_all_gather)
from .impls.communicate import (all_to_all, all_to_all_single, all_gather, zero_gather,
                                zero_scatter, spatial_split, reduce_scatter, allreduce_forward,
                                allreduce_backward)


class TutelDistributedOptimizer:
    """ZeRO-style wrapper: every non-expert parameter is flattened, zero-padded and sharded
    over ``group``; the wrapped optimizer updates only the local shard (plus this rank's expert
    parameters, which are never shared); ``step`` reduce-scatters gradients, steps, and
    all-gathers the updated shards back into the full parameters."""

    def __init__(self, params, group=None, average_shared=False):
        params = list(params)
        self.params = [p for p in params if not hasattr(p, '_tutel_expert')]
        self.expert_params = [p for p in params if hasattr(p, '_tutel_expert')]
        self.shapes = [p.shape for p in self.params]
        self.group = group
        self.average_shared = average_shared

    def chunk_param(self):
        self.virt_params = [
            zero_scatter(p.data, simple_split, group=self.group)[0].clone().requires_grad_(True)
            for p in self.params]

    def chunk_grad(self):
        denom = get_world_size(self.group) if self.average_shared else 1
        for shard, p in zip(self.virt_params, self.params):
            if getattr(p, 'grad', None) is None:
                continue
            g = p.grad.reshape(-1)
            if denom != 1:
                g = g / denom
            shard.grad, _ = zero_scatter(g, simple_reduce_scatter, group=self.group)

    def restore(self):
        for shard, p, shape in zip(self.virt_params, self.params, self.shapes):
            full = simple_all_gather(shard.data, group=self.group).view(-1)
            p.data = full[:shape.numel()].view(shape)

    def warp_local(self, local_optim, *args, **kwargs):
        self.chunk_param()
        self.local_optim = local_optim(self.virt_params + self.expert_params, *args, **kwargs)
        return self

    wrap_local = warp_local

    def zero_grad(self):
        for p in self.params + self.expert_params:
            if getattr(p, 'grad', None) is not None:
                p.grad.detach_()
                p.grad.zero_()

    def step(self):
        self.chunk_grad()
        self.local_optim.step()
        self.restore()
