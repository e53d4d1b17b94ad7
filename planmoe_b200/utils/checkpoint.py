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

Sharded experts (fewer experts than ranks: ``sharded_count = W / E`` ranks share one expert) hold a slice of
the HIDDEN dimension instead of whole experts: rank ``r`` owns slice ``r % sharded_count`` of expert
``r // sharded_count`` — ``batched_fc1_w [1, M, H/s]``, ``batched_fc1_bias [1, H/s]``, ``batched_fc2_w
[1, H/s, O]`` and the ``ceil(O/s)``-wide slice of ``batched_fc2_bias``.  Pass ``sharded_count`` (of the saved
world) to the helpers; they join the slices along the hidden dimension, and cut the hidden dimension again
when the new world also has more ranks than experts.
"""

import torch
import torch.distributed as dist


def is_expert_key(key, marker='experts.'):
    return key.startswith(marker) or ('.' + marker) in key


def _hidden_dim(key):
    """Which dimension of an FFN expert tensor is the hidden (or, for fc2's bias, the sliced output) dimension."""
    if key.endswith('batched_fc1_w'):
        return 2
    if key.endswith('batched_fc1_bias') or key.endswith('batched_fc2_w') or key.endswith('batched_fc2_bias'):
        return 1
    return None


def _join_shards(key, parts, sharded_count, out_dim=None):
    """``parts``: the tensors of ranks 0 .. W-1.  Returns the tensor of all experts, whole."""
    if sharded_count == 1:
        return torch.cat(parts, dim=0)
    dim = _hidden_dim(key)
    if dim is None:
        raise ValueError("%s: do not know how a sharded expert splits this tensor" % key)
    experts = []
    for e in range(len(parts) // sharded_count):
        whole = torch.cat(parts[e * sharded_count:(e + 1) * sharded_count], dim=dim)
        if key.endswith('batched_fc2_bias') and out_dim is not None:
            whole = whole[:, :out_dim]                      # slices are ceil(O / s) wide: drop the padding
        experts.append(whole)
    return torch.cat(experts, dim=0)


def _cut_shard(key, full, rank, world):
    """The tensor rank ``rank`` of ``world`` ranks holds, cut from the tensor of all experts."""
    n = full.size(0)
    if world <= n:
        if n % world:
            raise ValueError("%s: %d experts do not split evenly over %d ranks" % (key, n, world))
        per = n // world
        return full[rank * per:(rank + 1) * per].clone()
    if world % n:
        raise ValueError("%s: %d ranks cannot share %d experts evenly" % (key, world, n))
    s = world // n
    dim = _hidden_dim(key)
    if dim is None:
        raise ValueError("%s: do not know how a sharded expert splits this tensor" % key)
    e, j = rank // s, rank % s
    t = full[e:e + 1]
    size = t.size(dim)
    if key.endswith('batched_fc2_bias'):
        width = (size + s - 1) // s
        piece = t.narrow(dim, min(j * width, size), max(0, min(width, size - j * width)))
        if piece.size(dim) < width:                         # the last slice is padded to the common width
            pad = list(piece.shape)
            pad[dim] = width - piece.size(dim)
            piece = torch.cat([piece, piece.new_zeros(pad)], dim=dim)
        return piece.clone()
    if size % s:
        raise ValueError("%s: hidden size %d does not split over %d shard ranks" % (key, size, s))
    return t.narrow(dim, j * (size // s), size // s).clone()


def _out_dims(states):
    """{key prefix: output dim} from the fc2 weights, needed to un-pad the sliced fc2 bias."""
    return {k[:-len('batched_fc2_w')]: v.size(2) for k, v in states.items() if k.endswith('batched_fc2_w')}


def gather_expert_state(state, group=None, marker='experts.', sharded_count=1):
    """Join every expert tensor over the ranks of ``group`` (collective): whole experts along dim 0, the slices
    of sharded experts along their hidden dimension; other tensors are returned as they are.  Works on CPU
    (Gloo) and CUDA (NCCL) tensors."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return dict(state)
    world = dist.get_world_size(group)
    outs = _out_dims(state)
    out = {}
    for key in sorted(state):
        t = state[key]
        if is_expert_key(key, marker) and torch.is_tensor(t):
            parts = [torch.empty_like(t) for _ in range(world)]
            dist.all_gather(parts, t.contiguous(), group=group)
            out[key] = _join_shards(key, parts, sharded_count, outs.get(key[:-len('batched_fc2_bias')]))
        else:
            out[key] = t
    return out


def shard_expert_state(full_state, rank, world, marker='experts.'):
    """The state_dict of rank ``rank`` in a world of ``world`` ranks, cut from a full state_dict: whole experts
    when there are at least as many experts as ranks, otherwise a hidden-dimension slice of one expert."""
    out = {}
    for key, t in full_state.items():
        if is_expert_key(key, marker) and torch.is_tensor(t):
            out[key] = _cut_shard(key, t, rank, world)
        else:
            out[key] = t
    return out


def reshard_state_dicts(rank_states, new_world, marker='experts.', sharded_count=1):
    """``rank_states``: the state_dicts of ranks 0 .. W-1 of the old world, ``sharded_count`` ranks per expert
    there.  Returns the list of state_dicts for ``new_world`` ranks.  Replicated tensors are taken from rank 0."""
    outs = _out_dims(rank_states[0])
    full = {}
    for key, t in rank_states[0].items():
        if is_expert_key(key, marker) and torch.is_tensor(t):
            full[key] = _join_shards(key, [s[key] for s in rank_states], sharded_count,
                                     outs.get(key[:-len('batched_fc2_bias')]))
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


def load_sharded(module, prefix, saved_world=None, group=None, strict=True, marker='experts.', saved_sharded_count=1):
    """Load this rank's shard.  If the files were written by a world of another size (``saved_world``, with
    ``saved_sharded_count`` ranks per expert), every file is read and the expert tensors are re-cut for the
    current world."""
    ready = dist.is_available() and dist.is_initialized()
    rank = dist.get_rank(group) if ready else 0
    world = dist.get_world_size(group) if ready else 1
    saved_world = world if saved_world is None else int(saved_world)
    if saved_world == world:
        state = torch.load(_shard_path(prefix, rank, world), map_location='cpu')
    else:
        olds = [torch.load(_shard_path(prefix, r, saved_world), map_location='cpu') for r in range(saved_world)]
        state = reshard_state_dicts(olds, world, marker, saved_sharded_count)[rank]
    return module.load_state_dict(state, strict=strict)
