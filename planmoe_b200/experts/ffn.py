"""Batched two-layer FFN experts: ``y = act(x @ W1 + b1) @ W2 + b2`` for every local expert.

Reference: ``PlanMoE/experts/ffn.py:8-93``.  Parameter names, shapes and layout are the
checkpoint format and are kept exactly: ``batched_fc1_w [E_l, M, H]`` and
``batched_fc2_w [E_l, H, O]`` are input-major (``Linear.weight.T``), ``batched_fc1_bias
[E_l, H]``, ``batched_fc2_bias [E_l, ceil(O / sharded_count)]``.  Initial values are drawn,
expert by expert, from ``torch.nn.Linear``'s default init so a given seed reproduces the
reference's tensors.

On CUDA with bf16 parameters the two GEMMs run on the hand-written tcgen05 grouped GEMM of the
native extension (bias + activation in the epilogue); everything else uses ``torch.matmul``.
When an expert is sharded over ``sharded_count`` ranks (fewer experts than ranks) the hidden
dimension is split and the partial outputs are summed by the caller; ``b2`` is then added by
the first shard only.
"""

import os

import torch
import torch.nn.functional as F

_KNOWN_ACTS = {
    F.relu: 'relu', torch.relu: 'relu',
    F.gelu: 'gelu',
    F.silu: 'silu',
}


def activation_name(fn):
    """Name of a fusable activation ('relu' | 'gelu' | 'silu' | 'identity') or None."""
    if fn is None:
        return 'relu'
    if isinstance(fn, str):
        return fn if fn in ('relu', 'gelu', 'silu', 'identity') else None
    if isinstance(fn, torch.nn.ReLU):
        return 'relu'
    if isinstance(fn, torch.nn.GELU) and getattr(fn, 'approximate', 'none') == 'none':
        return 'gelu'
    if isinstance(fn, torch.nn.SiLU):
        return 'silu'
    if isinstance(fn, torch.nn.Identity):
        return 'identity'
    try:
        return _KNOWN_ACTS.get(fn)
    except TypeError:
        return None


_ACT_FNS = {'relu': F.relu, 'gelu': F.gelu, 'silu': F.silu, 'identity': lambda x: x}


class FusedExpertsNetwork(torch.nn.Module):
    def __init__(self, hidden_size_per_expert, activation_fn=None, activation_fn_with_self=None,
                 output_dim=None):
        super().__init__()
        self.skip_expert = (int(os.environ.get('SKIP_EXPERT', '0')) != 0)
        self.hidden_size_per_expert = hidden_size_per_expert
        self.output_dim = output_dim

        if activation_fn_with_self is not None:
            assert activation_fn is None, \
                "Option `activation_fn_with_self` has been specified, please keep exactly one of them."
            self.act_name = None
            self.activation_fn = lambda x: activation_fn_with_self(x, self)
        else:
            self.act_name = activation_name(activation_fn)
            if isinstance(activation_fn, str) or activation_fn is None:
                assert self.act_name is not None, "Unknown activation name: %s" % activation_fn
                activation_fn = _ACT_FNS[self.act_name]
            self.activation_fn = activation_fn

    def update(self, ctx):
        """Allocate the batched parameters for ``ctx`` (the owning MoE layer)."""
        shards = ctx.sharded_count
        if shards > 1:
            assert self.hidden_size_per_expert % shards == 0, \
                "Can't evenly divide hidden_size_per_expert (%d) to %d slices." % (
                    self.hidden_size_per_expert, shards)
        hidden = self.hidden_size_per_expert // shards
        model_dim, n_local = ctx.model_dim, ctx.num_local_experts
        self.output_dim = self.output_dim or model_dim
        bias2 = (self.output_dim + shards - 1) // shards

        w1 = torch.empty(n_local, model_dim, hidden)
        w2 = torch.empty(n_local, hidden, self.output_dim)
        b1 = torch.empty(n_local, hidden)
        b2 = torch.empty(n_local, bias2)
        for e in range(n_local):
            fc1 = torch.nn.Linear(model_dim, hidden)
            fc2 = torch.nn.Linear(hidden, self.output_dim)
            with torch.no_grad():
                w1[e].copy_(fc1.weight.t())
                b1[e].copy_(fc1.bias)
                w2[e].copy_(fc2.weight.t())
                b2[e].copy_(fc2.bias[:bias2])
        self.batched_fc1_w = torch.nn.Parameter(w1)
        self.batched_fc2_w = torch.nn.Parameter(w2)
        self.batched_fc1_bias = torch.nn.Parameter(b1)
        self.batched_fc2_bias = torch.nn.Parameter(b2)
        self.sharded_count = shards
        self.shard_rank = getattr(ctx, 'shard_rank', 0)

    def extra_repr(self):
        return 'model_dim=%d, hidden_size=%d, output_dim=%d, local_experts=%d' % (
            self.batched_fc1_w.size(1), self.batched_fc1_w.size(2),
            self.batched_fc2_w.size(2), self.batched_fc1_w.size(0))


    def fused_ok(self, x):
        return (x.is_cuda and x.dtype == torch.bfloat16 and self.act_name is not None
                and self.batched_fc1_w.dtype == torch.bfloat16 and self.sharded_count == 1
                and x.size(-1) % 64 == 0 and self.batched_fc1_w.size(2) % 64 == 0
                and self.batched_fc2_w.size(2) % 64 == 0
                and os.environ.get('PLANMOE_GEMM', 'tcgen05') == 'tcgen05')

    def forward(self, x, ctx=None):
        if self.skip_expert:
            return x
        w1, w2 = self.batched_fc1_w, self.batched_fc2_w
        b1, b2 = self.batched_fc1_bias, self.batched_fc2_bias
        if self.fused_ok(x):
            from ..ops import gemm
            return gemm.expert_ffn(x, w1, b1, w2, b2, self.act_name)

        zero_group = getattr(ctx, 'ffn_zero_group', None) if ctx is not None else None
        if zero_group is not None and not ctx.use_model_parallel:
            # 'data' sharding: this rank holds a slice of an expert's slots; rebuild the full expert
            # from the shards of its group (gradients flow back through a reduce-scatter).
            from ..impls.communicate import PrimAllgather

            def gather(t, dim):
                t = t.transpose(0, dim).contiguous()
                return PrimAllgather.apply(t, True, zero_group).transpose(0, dim)
            w1, b1, w2 = gather(w1, 2), gather(b1, 1), gather(w2, 1)
            b2 = gather(b2, 1)[:, :w2.size(2)]
            y = torch.matmul(self.activation_fn(torch.matmul(x, w1) + b1.unsqueeze(1)), w2)
            return y + b2.unsqueeze(1)

        y = torch.matmul(x, w1) + b1.unsqueeze(1)
        y = self.activation_fn(y)
        y = torch.matmul(y, w2)
        if self.sharded_count == 1:
            return y + b2.unsqueeze(1)
        # hidden-split shards: the caller sums partial outputs over the shard group; each shard
        # adds its slice of b2 into the matching output columns so the sum carries b2 once.
        width = b2.size(1)
        lo = self.shard_rank * width
        hi = min(lo + width, y.size(-1))
        if hi > lo:
            y = y.clone()
            y[..., lo:hi] += b2[:, :hi - lo].unsqueeze(1)
        return y


ExpertModule = FusedExpertsNetwork
