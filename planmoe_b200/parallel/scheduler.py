"""Adaptive pipeline-degree scheduler for the MoE layer.

The reference advertises an "adaptive optimal scheduling algorithm" (README.md:11,18) but ships only
a user-supplied chunk count (``a2a_ffn_overlap_degree``, PlanMoE/impls/moe_layer.py:53,228) and a
fixed issue order (PlanMoE/impls/overlap.py:59-74).  This module supplies the missing part:
``a2a_ffn_overlap_degree='auto'`` (or 0) makes the layer

  1. run ``warmup`` steps at degree 1,
  2. time ``samples`` whole steps (forward + backward + optimizer, measured on the device between
     consecutive forward entries) for every candidate degree,
  3. take the MAX over ranks of each candidate's median (one all-reduce, one host read), freeze
     the fastest degree — identical on every rank, which the capacity alignment requires — and
  4. store the decision in a JSON plan cache keyed by the layer's shape, world size, codec and
     comm algorithm, so later runs skip calibration.

The measurement costs no host synchronisation until the single read at the end of calibration.

The end of the module holds the analytic counterpart (a three-machine flow-shop model of the chunk
pipeline, ``predict_degree`` / ``codec_pays_off`` / ``rank_candidates``): it explains the measured
choice from per-stage times and orders candidates, but decisions are taken by measurement.
"""

import json
import os

import torch
import torch.distributed as dist

_CANDIDATES = (1, 2, 4, 8)


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


class AdaptiveScheduler:
    def __init__(self, key, group=None, candidates=_CANDIDATES, warmup=3, samples=4, use_cache=True):
        self.key, self.group = key, group
        self.candidates = [d for d in candidates if d <= 32]
        self.warmup, self.samples = warmup, samples
        self.use_cache = use_cache
        self.step = 0
        self.frozen = None
        self.events = []            # (degree, event at forward entry)
        self.report = None
        if use_cache:
            hit = _load_cache().get(key)
            if hit is not None and int(hit.get('degree', 0)) in self.candidates:
                self.frozen = int(hit['degree'])
                self.report = dict(hit, source='cache')

    @classmethod
    def for_layer(cls, layer):
        ex = layer.experts
        hidden = getattr(ex, 'hidden_size_per_expert', 0)
        key = 'M%d_H%s_E%d_W%d_%s_%s' % (layer.model_dim, hidden, layer.num_global_experts, layer.world_size,
                                         layer.compress_name, layer.comm_name)
        return cls(key, layer.group, use_cache=os.environ.get('PLANMOE_PLAN_CACHE_DISABLE', '0') != '1')

    # -- schedule -------------------------------------------------------------------------------
    def _plan_degree(self, step):
        if step < self.warmup:
            return self.candidates[0]
        i = (step - self.warmup) // (self.samples + 1)
        return self.candidates[i] if i < len(self.candidates) else None

    def next_degree(self):
        if self.frozen is not None:
            return self.frozen
        d = self._plan_degree(self.step)
        if d is None:
            self._decide()
            return self.frozen
        return d

    def begin_step(self, x):
        if self.frozen is not None:
            return
        if x.is_cuda:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
        else:
            import time
            ev = time.perf_counter()
        self.events.append((self._plan_degree(self.step), ev))

    def end_step(self, x):
        if self.frozen is None:
            self.step += 1

    # -- decision -------------------------------------------------------------------------------
    def _decide(self):
        times = {d: [] for d in self.candidates}
        for (d0, e0), (d1, e1) in zip(self.events[:-1], self.events[1:]):
            if d0 is None or d0 != d1:
                continue                     # first step at a new degree carries the switch cost
            if isinstance(e0, float):
                ms = (e1 - e0) * 1e3
            else:
                e1.synchronize()
                ms = e0.elapsed_time(e1)
            times[d0].append(ms)
        med = []
        for d in self.candidates:
            v = sorted(times[d][-self.samples:])
            med.append(v[len(v) // 2] if v else float('inf'))
        t = torch.tensor(med, dtype=torch.float64)
        if dist.is_available() and dist.is_initialized() and dist.get_world_size(self.group) > 1:
            dev = torch.device('cuda', torch.cuda.current_device()) if dist.get_backend(self.group) == 'nccl' else 'cpu'
            t = t.to(dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)
            t = t.cpu()
        best = int(torch.argmin(t))
        self.frozen = self.candidates[best]
        self.report = {'degree': self.frozen, 'ms': {str(d): float(v) for d, v in zip(self.candidates, t.tolist())},
                       'source': 'calibration'}
        self.events = []
        if self.use_cache:
            rank = dist.get_rank() if dist.is_available() and dist.is_initialized() else 0
            if rank == 0:
                cache = _load_cache()
                cache[self.key] = {'degree': self.frozen, 'ms': self.report['ms']}
                _store_cache(cache)


# ---------------------------------------------------------------------------------------------------
# Analytic pipeline model (decision support; the scheduler above decides by measurement)
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
# shrunken transfer beat the raw transfer.

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
