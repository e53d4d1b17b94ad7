"""Megatron-LM integration: command-line flags and the MoE replacement for a decoder layer's MLP.

The reference ships this as a patch against Megatron-LM ``core_r0.9.0``
(``PlanMoE/examples/megatron/schemoe_megatron.diff:28-37,54-101``): four flags
``--schemoe`` / ``--schemoe-overlap-degree`` / ``--schemoe-compress-name`` / ``--schemoe-comm-name``
and, when enabled, every decoder layer's ``mlp`` becomes a ``moe_layer`` (top-k linear gate in fp32
with gate noise 1.0, GELU FFN experts, ``param.allreduce = False`` on expert parameters so that the
data-parallel reducer skips them).  Here the same logic is importable code, and ``planmoe_megatron.diff`` next
to this file is the patch that makes Megatron call it (``git apply`` it in a ``core_r0.9.0`` checkout).
"""

import torch
import torch.nn.functional as F


def add_planmoe_args(parser):
    """Call from ``megatron/training/arguments.py`` (``_add_training_args`` or similar)."""
    group = parser.add_argument_group(title='planmoe')
    group.add_argument('--schemoe', action='store_true', help='Replace decoder MLPs by planmoe moe_layer.')
    group.add_argument('--schemoe-overlap-degree', default='1',
                       help="Pipeline chunk count (a2a_ffn_overlap_degree): an int or 'auto'.")
    group.add_argument('--schemoe-compress-name', type=str, default='no', choices=['no', 'zfp', 'int8', 'lz'])
    group.add_argument('--schemoe-comm-name', type=str, default='naive', choices=['naive', 'pipe', 'dd', 'hetu', 'nccl'])
    return parser


class PlanMoEMLP(torch.nn.Module):
    """Drop-in for Megatron's ``MLP`` / ``MoELayer`` module: ``forward(hidden) -> (output, bias)``."""

    def __init__(self, config, args=None, group=None):
        super().__init__()
        from planmoe_b200.moe import moe_layer
        degree = getattr(args, 'schemoe_overlap_degree', '1')
        degree = degree if degree == 'auto' else int(degree)
        experts_per_rank = max(1, int(getattr(config, 'num_moe_experts', 1) or 1) //
                               max(1, int(getattr(config, 'expert_model_parallel_size', 1) or 1)))
        self.moe = moe_layer(
            gate_type={'type': 'top', 'k': int(getattr(config, 'moe_router_topk', 2)), 'fp32_gate': True,
                       'gate_noise': 1.0, 'capacity_factor': float(getattr(config, 'moe_expert_capacity_factor', None) or 1.5)},
            model_dim=config.hidden_size,
            experts={'type': 'ffn', 'count_per_node': experts_per_rank,
                     'hidden_size_per_expert': config.ffn_hidden_size, 'activation_fn': F.gelu},
            scan_expert_func=lambda name, param: setattr(param, 'allreduce', False),
            group=group, a2a_ffn_overlap_degree=degree,
            compress_name=getattr(args, 'schemoe_compress_name', 'no'),
            comm_name=getattr(args, 'schemoe_comm_name', 'naive'))

    def forward(self, hidden_states):
        out = self.moe(hidden_states)
        self.l_aux = out.l_aux
        return out, None


def maybe_replace_mlp(layer, config, args, group=None):
    """Call at the end of ``TransformerLayer.__init__``: swaps ``layer.mlp`` when ``--schemoe`` is set."""
    if getattr(args, 'schemoe', False):
        layer.mlp = PlanMoEMLP(config, args, group)
    return layer


def wrap_model_provider(model_provider, args):
    """Wraps Megatron's ``model_provider`` (called from ``pretrain``): the model is built as usual, then the ``mlp``
    of every decoder layer is replaced by ``PlanMoEMLP``.  Its ``forward`` returns ``(output, None)`` like
    Megatron's MLP, so ``TransformerLayer.forward`` needs no change."""
    def provider(pre_process=True, post_process=True, **kwargs):
        try:
            model = model_provider(pre_process=pre_process, post_process=post_process, **kwargs)
        except TypeError:
            model = model_provider()
        config = getattr(model, 'config', None)
        for layer in model.decoder.layers:
            maybe_replace_mlp(layer, config if config is not None else layer.config, args)
        return model
    return provider
