"""fairseq integration helpers.

The reference patches fairseq (commit b5e7b25) so that every ``MOE``-th decoder layer's FFN becomes a
``moe_layer`` (top-2, dynamic capacity, one expert per GPU), collects the layers' ``l_aux`` through
``system.cache()`` and adds ``L_AUX_WT * sample_size * sum(l_aux)`` to the loss, and with
``NO_OVERFLOW=1`` zeroes non-finite gradients before the optimizer step
(``PlanMoE/examples/fairseq_moe/fairseq_patch.diff:41-54,82-84,103-106,119-128``).
These functions hold that logic; README.md next to this file shows where fairseq calls them.
"""

import os

import torch


def moe_every():
    """Env ``MOE``: every n-th decoder layer is MoE (0 = none)."""
    return int(os.environ.get('MOE', 0))


def build_ffn(layer_index, embed_dim, ffn_dim, activation_fn=None):
    """Return a ``moe_layer`` for MoE layers, or None (keep fairseq's dense fc1/fc2)."""
    n = moe_every()
    if n <= 0 or (layer_index + 1) % n != 0:
        return None
    from planmoe_b200.moe import moe_layer
    return moe_layer(
        gate_type={'type': 'top', 'k': 2, 'capacity_factor': 0.0, 'fp32_gate': True, 'gate_noise': 1.0},
        model_dim=embed_dim,
        experts={'type': 'ffn', 'count_per_node': 1, 'hidden_size_per_expert': ffn_dim,
                 'activation_fn': activation_fn or torch.nn.functional.gelu},
        scan_expert_func=lambda name, param: setattr(param, 'expert', True))


def ffn_forward(moe, x):
    """Run the MoE FFN and record its auxiliary loss in the process-wide cache."""
    from planmoe_b200 import system
    y = moe(x)
    system.cache().set(id(moe), y.l_aux)
    return y


def add_aux_loss(loss, sample_size):
    """``loss + L_AUX_WT * sample_size * sum(l_aux of all MoE layers)``; clears the cache."""
    from planmoe_b200 import system
    weight = float(os.environ.get('L_AUX_WT', 0.01))
    aux = [a for a in system.cache().get() if a is not None]
    system.cache().reset()
    if not aux:
        return loss
    return loss + weight * sample_size * sum(a.float() for a in aux)


def sanitize_grads(parameters):
    """Env ``NO_OVERFLOW=1``: replace non-finite gradient entries by zero (keeps fp16 runs alive)."""
    if int(os.environ.get('NO_OVERFLOW', 0)) == 0:
        return
    for p in parameters:
        if p.grad is not None:
            torch.nan_to_num_(p.grad, nan=0.0, posinf=0.0, neginf=0.0)
