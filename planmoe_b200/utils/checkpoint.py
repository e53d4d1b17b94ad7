"""Expert-shard checkpoint helpers.

A ``moe_layer`` state_dict holds the gate tensors (replicated on every rank) and this rank's expert
shard: ``experts.batched_fc1_w [E_local, M, H]``, ``experts.batched_fc2_w [E_local, H, O]``,
``experts.batched_fc1_bias [E_local, H]``, ``experts.batched_fc2_bias [E_local, O]`` — global expert
``e`` lives on rank ``e // E_local`` at index ``e % E_local``.  The reference has no save / load code of
its own (host trainers write per-rank files; ``PlanMoE/examples/megatron/train_schemoe.sh:80``); these
helpers keep that per-rank format and add what a change of world size needs:

  * ``gather_expert_state``   per-rank state_dict -> full state_dict (all experts), collective;
  * ``shard_expert_state``    full state_dict -> the shard of one rank of a world of any size;
  * ``reshard_state_dicts``   offline: the per-rank dicts of one world size -> those of another;
  * ``save_sharded`` / ``load_sharded``   one file per rank, ``<prefix>.rank<r>-of-<W>.pt``.

Keys are matched by prefix (default ``experts.``), so the helpers also work on the state_dict of a
whole model whose MoE layers sit under longer names (any key that contains ``.experts.`` or starts
with ``experts.`` is an expert tensor).
"""

import torch
import torch.distributed as dist


def is_expert_key(key, marker='experts.'):
    return key.startswith(marker) or ('.' + marker) in key


def gather_expert_state(state, group=None, marker='experts.'):
    """Concatenate every expert tensor over the ranks of ``group`` along dim 0 (collective); other
    tensors are returned as they are.  Works on CPU (Gloo) and CUDA (NCCL) tensors."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return dict(state)
    world = dist.get_world_size(group)
    out = {}
    for key in sorted(state):
        t = state[key]
        if is_expert_key(key, marker) and torch.is_tensor(t):
            parts = [torch.empty_like(t) for _ in range(world)]
            dist.all_gather(parts, t.contiguous(), group=group)
            out[key] = torch.cat(parts, dim=0)
        else:
            out[key] = t
    return out


def shard_expert_state(full_state, rank, world, marker='experts.'):
    """The state_dict of rank ``rank`` in a world of ``world`` ranks, cut from a full state_dict."""
    out = {}
    for key, t in full_state.items():
        if is_expert_key(key, marker) and torch.is_tensor(t):
            n = t.size(0)
            if n % world:
                raise ValueError("%s: %d experts do not split evenly over %d ranks" % (key, n, world))
            per = n // world
            out[key] = t[rank * per:(rank + 1) * per].clone()
        else:
            out[key] = t
    return out


def reshard_state_dicts(rank_states, new_world, marker='experts.'):
    """``rank_states``: the state_dicts of ranks 0 .. W-1 of the old world.  Returns the list of
    state_dicts for ``new_world`` ranks.  Replicated tensors are taken from rank 0."""
    full = {}
    for key, t in rank_states[0].items():
        if is_expert_key(key, marker) and torch.is_tensor(t):
            full[key] = torch.cat([s[key] for s in rank_states], dim=0)
        else:
            full[key] = t
    return [shard_expert_state(full, r, new_world, marker) for r in range(new_world)]


def _shard_path(prefix, rank, world):
    return '%s.rank%d-of-%d.pt' % (prefix, rank, world)


def save_sharded(module, prefix, group=None):
    """Write this rank's state_dict to ``<prefix>.rank<r>-of-<W>.pt``; returns the path."""
    ready = dist.is_available() and dist.is_initialized()
    rank = dist.get_rank(group) if ready else 0
    world = dist.get_world_size(group) if ready else 1
    path = _shard_path(prefix, rank, world)
    torch.save({k: v.detach().cpu() for k, v in module.state_dict().items()}, path)
    return path


def load_sharded(module, prefix, saved_world=None, group=None, strict=True, marker='experts.'):
    """Load this rank's shard.  If the files were written by a world of another size (``saved_world``),
    every file is read and the expert tensors are re-cut for the current world."""
    ready = dist.is_available() and dist.is_initialized()
    rank = dist.get_rank(group) if ready else 0
    world = dist.get_world_size(group) if ready else 1
    saved_world = world if saved_world is None else int(saved_world)
    if saved_world == world:
        state = torch.load(_shard_path(prefix, rank, world), map_location='cpu')
    else:
        olds = [torch.load(_shard_path(prefix, r, saved_world), map_location='cpu') for r in range(saved_world)]
        state = reshard_state_dicts(olds, world, marker)[rank]
    return module.load_state_dict(state, strict=strict)
