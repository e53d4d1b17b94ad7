"""Per-layer routing counters.

Off by default.  With ``layer.collect_stats = True`` (or env ``PLANMOE_STATS=1`` at construction) every
forward leaves in ``layer.last_stats``: tokens routed to each expert, tokens that found a slot and tokens
dropped for lack of capacity (per expert and in total), capacity, pipeline degree, comm algorithm, codec and
the bytes one dispatch all-to-all puts on the wire per rank.  Counters are device tensors computed with a
handful of tensor ops on the routing result: nothing synchronises the host until the caller reads them
(``as_python`` does, for logging).  The reference only has commented-out prints of the capacity and of the
per-expert token counts (``PlanMoE/impls/fast_dispatch.py:176-177,192-193``).
"""

import os

import torch


def enabled_by_env():
    return os.environ.get('PLANMOE_STATS', '0') not in ('0', '', 'false')


def routing_stats(indices, locations, num_experts, capacity):
    """``indices`` / ``locations``: ``[K, S]`` tensors or lists of K ``[S]`` tensors (expert id and slot
    of every pick; expert id < 0 marks no pick).  Returns a dict of device tensors."""
    idx = torch.stack(list(indices)) if isinstance(indices, (list, tuple)) else indices
    loc = torch.stack(list(locations)) if isinstance(locations, (list, tuple)) else locations
    idx, loc = idx.reshape(-1).long(), loc.reshape(-1).long()
    picked = idx >= 0
    safe = torch.where(picked, idx, torch.zeros_like(idx))
    routed = torch.zeros(num_experts, dtype=torch.long, device=idx.device).scatter_add_(0, safe, picked.long())
    kept_mask = picked & (loc >= 0) & (loc < capacity)
    kept = torch.zeros(num_experts, dtype=torch.long, device=idx.device).scatter_add_(0, safe, kept_mask.long())
    return {
        'tokens_routed_per_expert': routed,
        'tokens_kept_per_expert': kept,
        'tokens_dropped_per_expert': routed - kept,
        'tokens_dropped': (routed - kept).sum(),
        'slot_utilisation': kept.sum().float() / max(num_experts * int(capacity), 1),
    }


def wire_stats(num_global_experts, capacity, model_dim, elem_bytes, world, compress_name, comm_name, degree):
    raw = int(num_global_experts) * int(capacity) * int(model_dim) * int(elem_bytes)
    return {'capacity': int(capacity), 'degree': int(degree), 'comm': comm_name, 'codec': compress_name,
            'a2a_raw_bytes_per_rank': raw,
            'a2a_remote_bytes_per_rank': raw * (world - 1) // max(world, 1)}


def as_python(stats):
    """Copy of ``stats`` with tensors turned into Python numbers / lists (synchronises the host)."""
    out = {}
    for k, v in (stats or {}).items():
        if torch.is_tensor(v):
            out[k] = v.item() if v.numel() == 1 else v.tolist()
        else:
            out[k] = v
    return out
