"""fairseq integration helpers.

The reference patches fairseq (commit b5e7b25) so that every ``MOE``-th decoder layer's FFN becomes a
``moe_layer`` (top-2, dynamic capacity, one expert per GPU), collects the layers' ``l_aux`` through
``system.cache()`` and adds ``L_AUX_WT * sample_size * sum(l_aux)`` to the loss, and with
``NO_OVERFLOW=1`` zeroes non-finite gradients before the optimizer step
(``PlanMoE/examples/fairseq_moe/fairseq_patch.diff:41-54,82-84,103-106,119-128``).
These functions hold that logic; ``planmoe_fairseq.diff`` next to this file is the patch that makes fairseq call
them (``git apply`` it in a checkout of that commit).
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


def tag_layer_index(cfg, index):
    """Record which decoder layer is being built (``TransformerDecoderBase`` builds them in a comprehension)."""
    cfg.transformer_index = index
    return cfg


def build_ffn_for_layer(layer, cfg):
    """The MoE FFN of a ``TransformerDecoderLayerBase`` under construction, or None for a dense layer.  The
    experts' activation is the layer's activation dropout (and FFN layer norm), as in the dense branch."""
    index = int(getattr(cfg, 'transformer_index', 0))
    n = moe_every()
    if n <= 0 or (index + 1) % n != 0:
        return None
    assert not getattr(layer, 'quant_noise', 0), "Unhandled quant_noise > 0.0 for MoE layer."

    def act(x):
        x = layer.activation_dropout_module(layer.activation_fn(x))
        return x if layer.ffn_layernorm is None else layer.ffn_layernorm(x)
    return build_ffn(index, layer.embed_dim, cfg.decoder.ffn_embed_dim, act)


def ffn_forward(moe, x):
    """Run the MoE FFN and record (tokens, l_aux) in the process-wide cache for the loss."""
    from planmoe_b200 import system
    y = moe(x)
    if y.l_aux is not None and y.l_aux.requires_grad:
        system.cache().set(id(moe), (y.numel() // y.size(-1), y.l_aux))
    return y


def add_aux_loss(loss, sample_size=None):
    """``loss + L_AUX_WT * sum(tokens * l_aux of every MoE layer)``; clears the cache.  With ``sample_size`` given,
    that count weighs every layer instead of the layer's own token count."""
    from planmoe_b200 import system
    weight = float(os.environ.get('L_AUX_WT', 0.0))
    entries = [a for a in system.cache().get() if a is not None]
    system.cache().reset()
    if not entries or not weight:
        return loss
    total = None
    for entry in entries:
        tokens, aux = entry if isinstance(entry, tuple) else (sample_size or 1, entry)
        term = aux.float() * (weight * (sample_size if sample_size is not None else tokens))
        total = term if total is None else total + term
    return loss + total


def sanitize_grads(parameters):
    """Env ``NO_OVERFLOW=1``: replace non-finite gradient entries by zero (keeps fp16 runs alive)."""
    if int(os.environ.get('NO_OVERFLOW', 0)) == 0:
        return
    for p in parameters:
        if p.grad is not None:
            torch.nan_to_num_(p.grad, nan=0.0, posinf=0.0, neginf=0.0)
