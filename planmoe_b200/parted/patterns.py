"""The seven SPMD primitives a node can be computed with (``PlanMoE/parted/patterns.py:12-129``).

Each rule is a generator ``rule(sess, node, output_dim, group_size, rank)`` that yields
``(rank, source_dims, connectors)``: the sharding state every input must arrive in, and code
templates (with ``$`` standing for the tensor) for collectives on inputs (keyed by input index) or
on the output (key ``''``).

  BAR    pass-through: output sharded like the matching input dim (or everything replicated)
  FAR    contraction dim sharded, partial results all-reduced              -> replicated output
  RS     contraction dim sharded, partial results reduce-scattered         -> output sharded on dim
  SPLIT  replicated inputs, output sliced locally                          -> output sharded on dim
  AG     output computed sharded on dim i, then all-gathered               -> replicated output
  A2A    output computed sharded on dim i, then all-to-all to dim          -> output sharded on dim
  ZERO   like BAR with parameters stored ZeRO-sharded and gathered on use
"""

from .solver import register_primitive


def _replicated(dim):
    return dim == -1


def _partitioned(dim):
    return dim >= 0


def _grad_sync(sess, node, source_dims):
    """Replicated inputs of a sharded compute need their gradients all-reduced in backward."""
    return {i: sess.backend.link('$', -1, None, is_param=(node.inputs[i].op_type == 'param'))
            for i, d in source_dims.items() if _replicated(d)}


@register_primitive('BAR')
def pass_through(sess, node, output_dim, group_size, rank):
    if output_dim < -1:
        return
    source_dims, parted = node.parser.emit_dims_by_id(output_dim)
    if _replicated(output_dim) and parted == 0:
        yield (0, source_dims, {})
        return
    yield (0, source_dims, _grad_sync(sess, node, source_dims))


def _over_reduce_axes(sess, node, rank, out_link):
    if node.parser.reduce_type != '+':
        return
    for i, ax in enumerate(sorted(node.parser.get_reduce_axes())):
        if rank is not None and i != rank:
            continue
        try:
            source_dims, parted = node.parser.emit_dims_by_name(ax)
        except NotImplementedError:
            continue
        if parted == 0:
            continue
        conn = _grad_sync(sess, node, source_dims)
        conn[''] = out_link
        yield (i, source_dims, conn)


@register_primitive('FAR')
def fwd_allreduce(sess, node, output_dim, group_size, rank):
    if not _replicated(output_dim):
        return
    yield from _over_reduce_axes(sess, node, rank, sess.backend.link('$', None, -1))


@register_primitive('RS')
def fwd_reduce_scatter(sess, node, output_dim, group_size, rank):
    if not _partitioned(output_dim):
        return
    yield from _over_reduce_axes(sess, node, rank, sess.backend.link('$', None, output_dim))


@register_primitive('SPLIT')
def fwd_spatial_split(sess, node, output_dim, group_size, rank):
    if not _partitioned(output_dim):
        return
    source_dims, parted = node.parser.emit_dims_by_id(-1)
    yield (0, source_dims, {'': sess.backend.link('$', -1, output_dim)})


@register_primitive('AG')
def fwd_all_gather(sess, node, output_dim, group_size, rank):
    if not _replicated(output_dim):
        return
    for i in range(len(node.shape)):
        if rank is not None and i != rank:
            continue
        if node.shape[i] % group_size != 0:
            continue
        try:
            source_dims, parted = node.parser.emit_dims_by_id(i)
        except NotImplementedError:
            continue
        if parted == 0:
            continue
        conn = _grad_sync(sess, node, source_dims)
        conn[''] = sess.backend.link('$', i, -1)
        yield (i, source_dims, conn)


@register_primitive('A2A')
def fwd_all_to_all(sess, node, output_dim, group_size, rank):
    if not _partitioned(output_dim):
        return
    shape = node.shape
    if len(shape) < 2 or shape[output_dim] % group_size != 0:
        return
    for i in range(len(shape)):
        if rank is not None and i != rank:
            continue
        if i == output_dim or shape[i] % group_size != 0:
            continue
        try:
            source_dims, parted = node.parser.emit_dims_by_id(i)
        except NotImplementedError:
            continue
        if parted == 0:
            continue
        conn = _grad_sync(sess, node, source_dims)
        conn[''] = sess.backend.link('$', i, output_dim)
        yield (i, source_dims, conn)


@register_primitive('ZERO')
def zero_params(sess, node, output_dim, group_size, rank):
    if not _partitioned(output_dim):
        return
    source_dims, parted = node.parser.emit_dims_by_id(output_dim)
    if parted == 0:
        return
    conn, any_param = {}, False
    for i in list(source_dims):
        if not _replicated(source_dims[i]):
            continue
        if node.inputs[i].op_type == 'param':
            source_dims[i] = -2
            any_param = True
            conn[i] = sess.backend.link('$', -2, -1, output_shape=node.inputs[i].shape)
        else:
            conn[i] = sess.backend.link('$', -1, None, is_param=False)
    if any_param:
        yield (0, source_dims, conn)
