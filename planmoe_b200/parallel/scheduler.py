"""Adaptive scheduler of the MoE layer: pipeline degree, and on request the all-to-all algorithm.

The reference advertises an "adaptive optimal scheduling algorithm" (README.md:11,18) but ships only
a user-supplied chunk count (``a2a_ffn_overlap_degree``, PlanMoE/impls/moe_layer.py:53,228) and a
fixed issue order (PlanMoE/impls/overlap.py:59-74).  This module supplies the missing part.
``a2a_ffn_overlap_degree='auto'`` (or 0) and/or ``comm_name='auto'`` make the layer calibrate once, at its
first forward, and freeze a plan that is identical on every rank:

  * one rank: nothing crosses a link, every extra chunk is pure overhead, the plan is degree 1 without
    measuring;
  * rank 0 looks the layer up in a JSON plan cache and broadcasts hit-or-miss and the plan, so all ranks take
    the same branch (a rank-local lookup could hit on some ranks and miss on others, after which the
    ranks would run different chunk counts and mismatched collectives);
  * on a miss every candidate (degree x algorithm) is timed ON THE DEVICE: the layer's own forward +
    backward is enqueued ``samples`` times back to back behind a short delay kernel, so that the host runs
    ahead of the GPU and the CUDA events around each repetition bracket kernels that run without launch
    gaps (an eager training step whose host enqueue time exceeds its device time would otherwise measure
    the launch rate of the host, not the candidates).  The first repetitions absorb rank skew and are
    dropped, the faster half of the rest is averaged (noise only ever adds time), and the MAX over ranks of
    that is the candidate's cost;
  * the cheapest candidate wins, except that a larger degree must beat the best smaller one by more than
    ``margin`` (3 %): noise alone never moves the plan to more chunks;
  * the analytic flow-shop model at the end of the module is fed with the measured degree-1 stage split
    and orders the candidates; candidates it predicts to be more than 25 % behind are not measured, and
    its verdict on the codec (``codec_pays_off``) is recorded in the report when a codec is configured.

An integer ``a2a_ffn_overlap_degree`` still forces that degree, as in the reference.
"""

import json
import os
import time

import torch
import torch.distributed as dist

_CANDIDATES = (1, 2, 4, 8)
_COMM_CANDIDATES = ('naive', 'pipe', 'dd', 'hetu')


def _cache_path():
    return os.environ.get('PLANMOE_PLAN_CACHE',
                          os.path.join(os.path.expanduser('~'), '.cache', 'planmoe_b200', 'plans.json'))


def _load_cache():
    try:
        with open(_cache_path()) as f:
            return json.load(f)
    except Exception:
        return {}


def _store_cache(cache):
    path = _cache_path()
    try:
        os.makedirs(os.path.dirname(path), exist_ok=True)
        tmp = path + '.%d.tmp' % os.getpid()
        with open(tmp, 'w') as f:
            json.dump(cache, f, indent=1, sort_keys=True)
        os.replace(tmp, path)
    except Exception:
        pass


def robust_cost(values):
    """One number from repeated timings of the same work.  Timing noise is one-sided (interference only ever
    makes a repetition slower), so the estimate is the mean of the faster half, without the single fastest
    sample when there are at least five: slow outliers, however many, do not move it."""
    v = sorted(float(x) for x in values)
    if not v:
        return float('inf')
    lo = 1 if len(v) >= 5 else 0
    hi = max(lo + 1, (len(v) + 1) // 2)
    v = v[lo:hi]
    return sum(v) / len(v)


def choose(costs, margin=0.03):
    """Pick a plan from ``{(degree, comm): cost}``.  Candidates are visited by increasing degree (ties by
    name); a later one replaces the incumbent only if it is cheaper by more than ``margin``, so equal-cost
    candidates resolve to the fewest chunks and a noisy sample cannot flip the choice."""
    best = None
    for key in sorted(costs, key=lambda k: (k[0], str(k[1]))):
        c = costs[key]
        if c != c or c == float('inf'):
            continue
        if best is None or c < costs[best] * (1.0 - margin):
            best = key
    return best


class AdaptiveScheduler:
    def __init__(self, key, group=None, degrees=_CANDIDATES, comms=None, warmup=3, samples=10, margin=0.03,
                 use_cache=True):
        self.key, self.group = key, group
        self.degrees = [int(d) for d in degrees if d <= 32]
        self.comms = list(comms) if comms else [None]      # None: the layer's configured algorithm
        self.warmup, self.samples, self.margin = int(warmup), int(samples), float(margin)
        self.use_cache = use_cache
        self.frozen = None            # chosen degree
        self.frozen_comm = None       # chosen algorithm (None: the configured one)
        self.report = None

    @classmethod
    def for_layer(cls, layer, x=None, top_k=None, capacity_factor=None, degree_auto=True):
        ex = layer.experts
        hidden = getattr(ex, 'hidden_size_per_expert', 0)
        S = int(x.shape[0]) if x is not None else 0
        dt = str(x.dtype).replace('torch.', '') if x is not None else '?'
        key = 'M%d_H%s_E%d_W%d_S%d_k%s_cf%s_%s_%s_%s' % (
            layer.model_dim, hidden, layer.num_global_experts, layer.world_size, S, top_k, capacity_factor, dt,
            layer.compress_name, layer.comm_name)
        comms = _COMM_CANDIDATES if layer.comm_name == 'auto' else None
        degrees = _CANDIDATES if degree_auto else (int(layer.a2a_ffn_overlap_degree),)
        return cls(key, layer.group, degrees=degrees, comms=comms,
                   use_cache=os.environ.get('PLANMOE_PLAN_CACHE_DISABLE', '0') != '1')

    # -- collectives over the layer's group ---------------------------------------------------------
    def _world(self):
        if dist.is_available() and dist.is_initialized():
            return dist.get_world_size(self.group)
        return 1

    def _rank(self):
        if dist.is_available() and dist.is_initialized():
            return dist.get_rank(self.group)
        return 0

    def _bcast_obj(self, obj):
        if self._world() == 1:
            return obj
        box = [obj]
        src = dist.get_global_rank(self.group, 0) if self.group is not None else 0
        dist.broadcast_object_list(box, src=src, group=self.group)
        return box[0]

    def _max_over_ranks(self, values, device):
        t = torch.tensor(values, dtype=torch.float64)
        if self._world() > 1:
            dev = device if (device.type == 'cuda' and dist.get_backend(self.group) == 'nccl') else torch.device('cpu')
            t = t.to(dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)
            t = t.cpu()
        return t.tolist()

    # -- the decision -----------------------------------------------------------------------------
    def _freeze(self, degree, comm, report):
        self.frozen, self.frozen_comm = int(degree), comm
        self.report = report

    def resolve(self, run_candidate, device, allowed_degree=lambda d: True, stage_split=None, codec_info=None):
        """Freeze a plan (collective over the group; returns ``(degree, comm)``).

        ``run_candidate(degree, comm)`` enqueues ONE forward + backward of the layer on the current data with
        that plan and returns nothing; it must not synchronise.  ``stage_split()`` (optional) returns
        ``(t_send, t_ffn, t_return)`` measured at degree 1 for the analytic model."""
        if self.frozen is not None:
            return self.frozen, self.frozen_comm
        degrees = [d for d in self.degrees if allowed_degree(d)] or [1]
        if self._world() == 1:
            # a single rank has nothing to overlap: more chunks only add tile and flag overhead
            self._freeze(min(degrees), self.comms[0], {'degree': min(degrees), 'source': 'single rank'})
            return self.frozen, self.frozen_comm

        hit = None
        if self.use_cache and self._rank() == 0:
            hit = _load_cache().get(self.key)
            if hit is not None and (int(hit.get('degree', 0)) not in degrees or
                                    (hit.get('comm') not in self.comms)):
                hit = None
        hit = self._bcast_obj(hit)
        if hit is not None:
            self._freeze(hit['degree'], hit.get('comm'), dict(hit, source='cache'))
            return self.frozen, self.frozen_comm

        cands = [(d, c) for c in self.comms for d in degrees]
        pred = None
        if stage_split is not None and len(degrees) > 1:
            try:
                t_send, t_ffn, t_return = stage_split()
                _, pred = predict_degree(t_send, t_ffn, t_return, degrees, per_chunk_overhead=0.01 * (t_send + t_ffn + t_return))
                floor = min(pred.values())
                keep = {d for d in degrees if pred[d] <= 1.25 * floor or d == min(degrees)}
                keep = self._bcast_obj(sorted(keep))            # every rank measures the same candidates
                cands = [(d, c) for (d, c) in cands if d in keep]
            except Exception:
                pred = None

        raw = {}
        for key in cands:
            raw[key] = self._time_candidate(run_candidate, key, device)
        order = sorted(raw)
        maxed = self._max_over_ranks([raw[k] for k in order], device)
        costs = dict(zip(order, maxed))
        best = choose(costs, self.margin)
        if best is None:
            best = (min(degrees), self.comms[0])
        report = {'degree': best[0], 'comm': best[1], 'source': 'calibration', 'samples': self.samples,
                  'margin': self.margin,
                  'ms': {('%d' % d if c is None else '%d/%s' % (d, c)): round(v, 5) for (d, c), v in sorted(costs.items(), key=lambda kv: (kv[0][0], str(kv[0][1])))}}
        if pred is not None:
            report['model_ms'] = {str(d): round(v, 5) for d, v in pred.items()}
        if codec_info is not None:
            report['codec'] = codec_info
        self._freeze(best[0], best[1], report)
        if self.use_cache and self._rank() == 0:
            cache = _load_cache()
            cache[self.key] = {'degree': best[0], 'comm': best[1], 'ms': report['ms']}
            _store_cache(cache)
        return self.frozen, self.frozen_comm

    def _time_candidate(self, run_candidate, key, device):
        """Device time of one forward + backward under plan ``key`` (ms, ``robust_cost`` over ``samples`` repetitions)."""
        degree, comm = key
        n = self.warmup + self.samples
        if device.type != 'cuda':
            times = []
            for i in range(n):
                t0 = time.perf_counter()
                run_candidate(degree, comm)
                times.append((time.perf_counter() - t0) * 1e3)
            return robust_cost(times[self.warmup:])
        from ..ops import native
        lib = native.maybe_lib()
        run_candidate(degree, comm)                          # allocations, tensor maps and caches of this plan
        torch.cuda.synchronize(device)
        events = [torch.cuda.Event(enable_timing=True) for _ in range(n + 1)]
        if lib is not None and hasattr(lib, 'delay'):
            lib.delay(int(2_000_000 + 600_000 * n))          # ns: the host gets ahead of the device
        events[0].record()
        for i in range(n):
            run_candidate(degree, comm)
            events[i + 1].record()
        events[-1].synchronize()
        times = [events[i].elapsed_time(events[i + 1]) for i in range(n)]
        return robust_cost(times[self.warmup:])


# ---------------------------------------------------------------------------------------------------
# Analytic pipeline model
# ---------------------------------------------------------------------------------------------------
# A layer split into d chunks is a three-machine flow shop with d identical jobs: the dispatch link
# (send of a chunk), the SMs (expert FFN of a chunk) and the return link (combine send of a chunk).
# With per-chunk times a, b, c and a fixed cost per chunk o (flag round trips, tile quantisation, extra
# launches) the makespan of such a shop is
#
#       T(d) = a + b + c + (d - 1) * max(a, b, c) + d * o,      a = t_send / d, b = t_ffn / d, c = t_return / d.
#
# d = 1 is the unpipelined sum; a large d approaches the slowest resource plus the per-chunk costs.  The
# same arithmetic says whether a codec pays for itself on a link: it does when encode + decode + the
# shrunken transfer beat the raw transfer.  The scheduler uses the model to skip hopeless candidates before
# measuring and to annotate its report; the decision itself is taken by measurement.

def flow_shop_makespan(t_send, t_ffn, t_return, degree, per_chunk_overhead=0.0):
    """Predicted time of one pipelined pass (any unit) for ``degree`` chunks."""
    d = max(int(degree), 1)
    a, b, c = t_send / d, t_ffn / d, t_return / d
    return a + b + c + (d - 1) * max(a, b, c) + d * per_chunk_overhead


def predict_degree(t_send, t_ffn, t_return, candidates=_CANDIDATES, per_chunk_overhead=0.0):
    """The candidate degree with the smallest predicted makespan, and the predictions."""
    pred = {d: flow_shop_makespan(t_send, t_ffn, t_return, d, per_chunk_overhead) for d in candidates}
    best = min(candidates, key=lambda d: (pred[d], d))
    return best, pred


def codec_pays_off(t_encode, t_decode, t_transfer_raw, ratio):
    """True when compressing a payload by ``ratio`` shortens its trip: encode + decode + transfer / ratio
    against the raw transfer (all in the same unit)."""
    if ratio <= 1.0:
        return False
    return t_encode + t_decode + t_transfer_raw / ratio < t_transfer_raw


def rank_candidates(stage_us, candidates=_CANDIDATES, per_chunk_overhead_us=3.0):
    """Order candidate degrees by the model, from stage times as reported by ``utils.stage_timer.summary()``
    at degree 1 (keys containing 'dispatch', 'gemm' and 'combine'); stages it cannot find count as zero."""
    def pick(word):
        return sum(v['median_us'] if isinstance(v, dict) else float(v) for k, v in stage_us.items() if word in k)
    t_send, t_ffn, t_return = pick('dispatch'), pick('gemm'), pick('combine')
    _, pred = predict_degree(t_send, t_ffn, t_return, candidates, per_chunk_overhead_us)
    return sorted(candidates, key=lambda d: (pred[d], d)), pred
