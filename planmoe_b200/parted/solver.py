"""Search over SPMD sharding plans.

Counterpart of ``PlanMoE/parted/solver.py:9-144``: a registry of parallel primitives and
``solve_partition``.  Every node of the graph may be replicated (-1), ZeRO-sharded (-2, parameters
only) or partitioned on one of its dims (>= 0).  For the final node and every admissible output
state the solver returns the cheapest consistent assignment ``{node: (state, "PRIM:rank")}``.

Search: states of nodes with several consumers are enumerated; given those, the remaining graph is
a tree and is solved bottom-up by dynamic programming.  Candidate plans are priced by an analytic
model (FLOPs at the measured GEMM rate of the sharded compute + collective bytes at NVLink bus
bandwidth + a per-collective latency); with ``evaluate='run'`` the ``top_n`` cheapest complete
plans are compiled and executed and the measured step time decides (the reference executes every
partial candidate, one process launch each).
"""

import itertools
import json
import sys

spmd_primitives_dict = dict()

# pricing constants (B200, measured on this pool): bf16 GEMM TFLOP/s, NVLink GB/s per direction
PEAK_FLOPS = 1.4e15
LINK_BYTES = 7.7e11
LATENCY_S = 12e-6


def register_primitive(name=None):
    if not name:
        name = 'custom_%d' % len(spmd_primitives_dict)

    def deco(func):
        assert name not in spmd_primitives_dict, "Parallel Pattern with name `%s` already exists." % name
        spmd_primitives_dict[name] = func
        return func
    return deco


def _bytes(node):
    width = {'float64': 8, 'float32': 4, 'float16': 2, 'bfloat16': 2, 'int64': 8, 'int32': 4}.get(str(node.dtype), 4)
    n = 1
    for s in node.shape:
        n *= int(s)
    return n * width


def comm_cost(kind, nbytes, group):
    """Seconds for one collective on `nbytes` (full, unsharded tensor) over `group` ranks."""
    if group <= 1 or kind is None:
        return 0.0
    frac = (group - 1) / group
    vol = {'allreduce': 2 * frac * nbytes, 'reduce_scatter': frac * nbytes, 'all_gather': frac * nbytes,
           'all_to_all': frac * nbytes / group, 'split': 0.0, 'bwd_allreduce': 2 * frac * nbytes,
           'zero_gather': 2 * frac * nbytes}[kind]
    return LATENCY_S + vol / LINK_BYTES


def convert_cost(node, src, dst, group):
    """Cost of re-laying out `node` from state src to state dst (what backend.link emits)."""
    if src == dst:
        return 0.0
    nb = _bytes(node)
    if src == -2:
        return comm_cost('zero_gather', nb, group) + (0.0 if dst == -1 else 0.0)
    if src == -1:
        return comm_cost('split', nb, group)
    if dst == -1:
        return comm_cost('all_gather', nb, group)
    return comm_cost('all_to_all', nb, group)


def _admissible_states(node, group, split_pref):
    if node.name in split_pref:
        return [split_pref[node.name]]
    if group == 1:
        return [-1]
    states = [-1]
    if node.op_type == 'param':
        states.append(-2)
    states += [d for d in range(len(node.shape)) if node.shape[d] % group == 0]
    return states


def solve_partition(sess, compute_groups, input_nodes, split_pref, kwargs):
    group = kwargs['spmd_nodes']
    evaluate = kwargs.get('evaluate', 'model')
    top_n = int(kwargs.get('top_n', 3))
    compute_nodes = [n for members, _ in compute_groups for n in members]
    last = compute_nodes[-1]
    consumers = {}
    for n in compute_nodes:
        for i in n.inputs:
            consumers[i.name] = consumers.get(i.name, 0) + 1
    shared = [n for n in list(input_nodes) + compute_nodes if consumers.get(n.name, 0) > 1]
    by_name = {n.name: n for n in list(input_nodes) + compute_nodes}

    shared_states = [_admissible_states(n, group, split_pref) for n in shared]
    combos = list(itertools.product(*shared_states)) if shared else [()]
    if len(combos) > 4096:
        combos = combos[:4096]

    results = {}          # final state -> (cost, config)

    for combo in combos:
        fixed = {n.name: s for n, s in zip(shared, combo)}
        table = {}        # node name -> {state: (cost, config)}
        for n in input_nodes:
            table[n.name] = {s: (0.0, {n.name: (s, '')}) for s in _admissible_states(n, group, split_pref)
                             if fixed.get(n.name, s) == s}
        ok = True
        for n in compute_nodes:
            table[n.name] = {}
            for state in _admissible_states(n, group, split_pref):
                if fixed.get(n.name, state) != state:
                    continue
                best = None
                for key, rule in spmd_primitives_dict.items():
                    try:
                        options = list(rule(sess, n, state, group, None))
                    except NotImplementedError:
                        continue
                    for rank, source_dims, connectors in options:
                        cost = n.flops / PEAK_FLOPS / (group if _is_sharded_compute(state, source_dims) else 1)
                        cfg = {n.name: (state, '%s:%d' % (key, rank))}
                        feasible = True
                        for idx, want in source_dims.items():
                            inp = n.inputs[idx]
                            choices = table.get(inp.name, {})
                            pick = None
                            for have, (c0, cfg0) in choices.items():
                                c = c0 + convert_cost(inp, have, want, group)
                                if have == -2 and want != -2 and inp.op_type != 'param':
                                    continue
                                if pick is None or c < pick[0]:
                                    pick = (c, cfg0)
                            if pick is None:
                                feasible = False
                                break
                            merged = _merge(cfg, pick[1])
                            if merged is None:
                                feasible = False
                                break
                            cfg = merged
                            cost += pick[0] if consumers.get(inp.name, 0) <= 1 else pick[0] / consumers[inp.name]
                            if idx in connectors and connectors[idx]:
                                cost += comm_cost('bwd_allreduce', _bytes(inp), group) if kwargs.get('run_mode') == 'train' else 0.0
                        if not feasible:
                            continue
                        out_comm = connectors.get('', '')
                        if out_comm:
                            kind = ('allreduce' if 'allreduce_forward' in out_comm else
                                    'reduce_scatter' if 'reduce_scatter' in out_comm else
                                    'all_gather' if 'all_gather' in out_comm else
                                    'all_to_all' if 'all_to_all' in out_comm else 'split')
                            cost += comm_cost(kind, _bytes(n), group)
                        if best is None or cost < best[0]:
                            best = (cost, cfg)
                if best is not None:
                    table[n.name][state] = best
            if not table[n.name]:
                ok = False
                break
        if not ok:
            continue
        for state, (cost, cfg) in table[last.name].items():
            if state not in results or cost < results[state][0]:
                results[state] = (cost, cfg)

    if evaluate == 'run' and results:
        ranked = sorted(results.items(), key=lambda kv: kv[1][0])[:top_n]
        measured = {}
        for state, (_, cfg) in ranked:
            full = _complete(cfg, by_name)
            prog = last.compile(full, **kwargs)
            print('>> Try final state %s, config = %s' % (state, json.dumps(full)))
            sys.stdout.flush()
            t = prog.execute().get('step_time', float('inf'))
            measured[state] = (t, full)
        results = measured
    else:
        results = {s: (c, _complete(cfg, by_name)) for s, (c, cfg) in results.items()}

    return [(dim, results.get(dim)) for dim in range(-1, len(last.shape))]


def _is_sharded_compute(state, source_dims):
    return state >= 0 or any(d >= 0 for d in source_dims.values())


def _merge(a, b):
    out = dict(a)
    for k, v in b.items():
        if k in out and out[k][0] != v[0]:
            return None
        out.setdefault(k, v)
    return out


def _complete(cfg, by_name):
    """Every node gets an entry (unreferenced inputs default to replicated)."""
    full = {k: [v[0], v[1]] for k, v in cfg.items()}
    for name in by_name:
        full.setdefault(name, [-1, ''])
    return full
