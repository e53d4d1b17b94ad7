"""Host-side utilities that need no GPU: stage timers when disabled, the benchmark's clock sampler
parsing, the CUDA-graph helper's import surface."""

import importlib
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_stage_timer_is_a_noop_when_disabled():
    from planmoe_b200.utils import stage_timer
    stage_timer.enable(False)
    stage_timer.reset()
    with stage_timer.stage('anything') as s:
        assert s.start is None
    assert stage_timer.summary() == {}
    assert not stage_timer.enabled()


def test_graph_helper_imports_without_cuda():
    mod = importlib.import_module('planmoe_b200.utils.graphs')
    assert hasattr(mod, 'GraphedSteps')


def test_bench_reference_arm_prints_unavailable_line():
    out = subprocess.run([sys.executable, os.path.join(ROOT, 'bench.py'), '--impl', 'reference'],
                         capture_output=True, text=True, timeout=120)
    assert out.returncode == 0
    rec = json.loads(out.stdout.strip().splitlines()[-1])
    assert rec['impl'] == 'reference' and rec['unavailable']


def test_clock_sampler_without_nvml_or_gpu_reports_no_samples():
    sys.path.insert(0, ROOT)
    bench = importlib.import_module('bench')
    s = bench.ClockSampler(0, None)
    s.start()
    res = s.stop()
    assert set(res) >= {'sm_mhz', 'sm_max_mhz', 'reasons', 'samples'}
