"""Per-stage device timers and NVTX ranges for the MoE pipeline.

Off by default and free when off (one attribute test per stage, no event, no host sync).  With
``PLANMOE_STAGE_TIMERS=1`` (or ``enable(True)``) every pipeline stage of the fused path is bracketed
by CUDA events recorded on the launching stream and by an NVTX range named after the stage;
``summary()`` synchronises once and returns the median duration of every stage in microseconds.
Because the stages of one step are enqueued on one stream, the time of a stage includes whatever
that stage waited for (a flag from a peer, a ring slot), which is what a pipeline schedule needs.

The reference only has a whole-step timer around its benchmark loop and an unused torch.profiler
handler (``PlanMoE/examples/pre_test.py:20-44,178-189``) and ``system.record_time``
(``PlanMoE/system.py:72-78``).
"""

import os
import statistics
from collections import OrderedDict

import torch

_ENABLED = os.environ.get('PLANMOE_STAGE_TIMERS', '0') not in ('0', '', 'false')
_RECORDS = OrderedDict()          # stage name -> list of (start event, end event)
_MAX_SAMPLES = 4096


def enabled():
    return _ENABLED


def enable(flag=True):
    global _ENABLED
    _ENABLED = bool(flag)


def reset():
    _RECORDS.clear()


class _Stage:
    __slots__ = ('name', 'start')

    def __init__(self, name):
        self.name = name
        self.start = None

    def __enter__(self):
        if _ENABLED and torch.cuda.is_available():
            torch.cuda.nvtx.range_push(self.name)
            self.start = torch.cuda.Event(enable_timing=True)
            self.start.record()
        return self

    def __exit__(self, *exc):
        if self.start is not None:
            end = torch.cuda.Event(enable_timing=True)
            end.record()
            torch.cuda.nvtx.range_pop()
            rec = _RECORDS.setdefault(self.name, [])
            if len(rec) < _MAX_SAMPLES:
                rec.append((self.start, end))
        return False


def stage(name):
    """``with stage('dispatch+gemm1'): ...`` — a no-op context unless timers are enabled."""
    return _Stage(name)


def summary(skip=0):
    """{stage: {'median_us', 'min_us', 'n'}} over the recorded samples (first ``skip`` dropped)."""
    if not _RECORDS:
        return {}
    torch.cuda.synchronize()
    out = OrderedDict()
    for name, rec in _RECORDS.items():
        us = [s.elapsed_time(e) * 1e3 for s, e in rec[skip:]]
        if us:
            out[name] = {'median_us': round(statistics.median(us), 1), 'min_us': round(min(us), 1), 'n': len(us)}
    return out
