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


def test_expert_shards_reshard_between_world_sizes(tmp_path):
    import torch
    from planmoe_b200.utils import checkpoint as ck
    torch.manual_seed(0)
    E, M, H = 8, 6, 10
    full = {'gates.0.wg.weight': torch.randn(E, M), 'experts.batched_fc1_w': torch.randn(E, M, H),
            'experts.batched_fc2_w': torch.randn(E, H, M), 'experts.batched_fc1_bias': torch.randn(E, H),
            'experts.batched_fc2_bias': torch.randn(E, M), 'decoder.layers.1.moe.experts.batched_fc1_w': torch.randn(E, M, H)}
    four = [ck.shard_expert_state(full, r, 4) for r in range(4)]
    assert four[1]['experts.batched_fc1_w'].shape == (2, M, H)
    assert torch.equal(four[3]['experts.batched_fc1_w'], full['experts.batched_fc1_w'][6:8])
    assert torch.equal(four[2]['gates.0.wg.weight'], full['gates.0.wg.weight'])          # replicated
    assert torch.equal(four[1]['decoder.layers.1.moe.experts.batched_fc1_w'],
                       full['decoder.layers.1.moe.experts.batched_fc1_w'][2:4])
    two = ck.reshard_state_dicts(four, 2)
    eight = ck.reshard_state_dicts(two, 8)
    back = ck.reshard_state_dicts(eight, 4)
    for a, b in zip(four, back):
        for k in a:
            assert torch.equal(a[k], b[k]), k
    one = ck.reshard_state_dicts(four, 1)[0]
    for k in full:
        assert torch.equal(one[k], full[k])
    import pytest
    with pytest.raises(ValueError):
        ck.shard_expert_state(full, 0, 3)


def test_sharded_save_and_load_round_trip_single_rank(tmp_path):
    import torch
    from planmoe_b200 import moe
    from planmoe_b200.utils import checkpoint as ck

    def make(seed):
        return moe.moe_layer(gate_type={'type': 'top', 'k': 2}, model_dim=16,
                             experts={'type': 'ffn', 'count_per_node': 4, 'hidden_size_per_expert': 32,
                                      'activation_fn': 'relu'}, seeds=(seed, seed + 1, seed + 2))
    a, b = make(1), make(7)
    prefix = str(tmp_path / 'ckpt')
    ck.save_sharded(a, prefix)
    ck.load_sharded(b, prefix)
    for (ka, va), (kb, vb) in zip(a.state_dict().items(), b.state_dict().items()):
        assert ka == kb and torch.equal(va, vb)
    x = torch.randn(32, 16)
    assert torch.equal(a(x), b(x))


def test_routing_counters_on_the_cpu_path():
    import torch
    from planmoe_b200 import moe
    from planmoe_b200.utils import metrics
    torch.manual_seed(0)
    layer = moe.moe_layer(gate_type={'type': 'top', 'k': 2, 'capacity_factor': 0.5}, model_dim=16,
                          experts={'type': 'ffn', 'count_per_node': 4, 'hidden_size_per_expert': 32,
                                   'activation_fn': 'relu'}, seeds=(1, 2, 3))
    x = torch.randn(64, 16)
    layer(x)
    assert 'tokens_dropped' not in layer.last_stats                      # off by default
    layer.collect_stats = True
    layer(x)
    st = metrics.as_python(layer.last_stats)
    assert st['path'] == 'generic' and st['codec'] == 'no' and st['degree'] == 1
    assert sum(st['tokens_routed_per_expert']) == 2 * 64                  # every token picks two experts
    assert all(k <= st['capacity'] for k in st['tokens_kept_per_expert'])
    assert st['tokens_dropped'] == sum(st['tokens_routed_per_expert']) - sum(st['tokens_kept_per_expert'])
    assert st['tokens_dropped'] > 0                                       # capacity factor 0.5 must drop some
    assert st['a2a_raw_bytes_per_rank'] == 4 * st['capacity'] * 16 * 4
    assert 0.0 < st['slot_utilisation'] <= 1.0


_JIT_SRC = '''
extern "C" __global__ void scale_by(float* __restrict__ x, int n) {
  // [thread_extent] blockIdx.x = 4
  // [thread_extent] threadIdx.x = 256
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) x[i] *= @factor@;
}
'''


def test_user_kernels_compile_for_sm100a_without_a_gpu_nvrtc_and_nvcc(monkeypatch):
    """Both compilation routes of the JIT engine produce an sm_100a cubin on a machine without a GPU."""
    from planmoe_b200 import jit
    for use_nvrtc in ('1', '0'):
        monkeypatch.setenv('USE_NVRTC', use_nvrtc)
        fn = jit.create_cuda_kernel(_JIT_SRC, {'factor': '2.0f'})
        size = int(fn.compile())
        assert size > 1000, (use_nvrtc, size)
    monkeypatch.setenv('USE_NVRTC', '0')
    bad = jit.create_cuda_kernel('extern "C" __global__ void broken(float* x) { x[0] = undefined_symbol; }')
    import pytest
    with pytest.raises(RuntimeError, match='nvcc failed'):
        bad.compile()


def test_pipeline_model_of_the_scheduler():
    from planmoe_b200.parallel import scheduler as sc
    # link-bound layer: chunking hides the FFN behind the transfers
    assert sc.flow_shop_makespan(80., 100., 80., 1) == 260.
    assert sc.flow_shop_makespan(80., 100., 80., 4) == 20. + 25. + 20. + 3 * 25.
    best, pred = sc.predict_degree(80., 100., 80., (1, 2, 4, 8), per_chunk_overhead=0.)
    assert best == 8 and pred[8] < pred[4] < pred[2] < pred[1]
    # a per-chunk cost makes deep pipelines lose again
    best, pred = sc.predict_degree(80., 100., 80., (1, 2, 4, 8), per_chunk_overhead=12.)
    assert best in (2, 4) and pred[8] > pred[best]
    # nothing to overlap: degree 1 wins as soon as chunks cost anything
    assert sc.predict_degree(0., 100., 0., (1, 2, 4, 8), per_chunk_overhead=1.)[0] == 1
    assert sc.codec_pays_off(10., 10., 100., 2.0) and not sc.codec_pays_off(30., 30., 100., 2.0)
    assert not sc.codec_pays_off(0., 0., 100., 1.0)
    order, pred = sc.rank_candidates({'fwd.dispatch': {'median_us': 80.}, 'fwd.gemm1': 60., 'fwd.gemm2': 40.,
                                      'fwd.combine_push': {'median_us': 80.}})
    assert order[0] in (4, 8) and set(order) == {1, 2, 4, 8}


def test_checkpoint_reshards_sharded_experts_along_the_hidden_dim():
    """Two experts on four ranks (two ranks per expert, hidden dim split) -> two ranks (whole experts) -> eight ranks
    (four slices per expert) and back: every tensor survives, fc2's sliced bias included (odd output dim)."""
    import torch
    from planmoe_b200.utils import checkpoint as ck
    E, M, H, O = 2, 6, 8, 5
    torch.manual_seed(0)
    full = {'gates.0.wg.weight': torch.randn(E, M),
            'experts.batched_fc1_w': torch.randn(E, M, H), 'experts.batched_fc1_bias': torch.randn(E, H),
            'experts.batched_fc2_w': torch.randn(E, H, O), 'experts.batched_fc2_bias': torch.randn(E, O)}
    four = [ck.shard_expert_state(full, r, 4) for r in range(4)]
    assert four[1]['experts.batched_fc1_w'].shape == (1, M, H // 2)
    assert four[1]['experts.batched_fc2_w'].shape == (1, H // 2, O)
    assert four[3]['experts.batched_fc2_bias'].shape == (1, 3)            # ceil(5 / 2), zero-padded
    assert torch.equal(four[2]['experts.batched_fc1_bias'], full['experts.batched_fc1_bias'][1:2, :H // 2])
    two = ck.reshard_state_dicts(four, 2, sharded_count=2)
    for r in range(2):
        for k in full:
            want = full[k][r:r + 1] if k.startswith('experts.') else full[k]
            assert torch.equal(two[r][k], want), (r, k)
    eight = ck.reshard_state_dicts(four, 8, sharded_count=2)
    assert eight[5]['experts.batched_fc1_w'].shape == (1, M, H // 4)
    back = ck.reshard_state_dicts(eight, 4, sharded_count=4)
    for r in range(4):
        for k in full:
            assert torch.equal(back[r][k], four[r][k]), (r, k)
    import pytest
    with pytest.raises(ValueError):
        ck.shard_expert_state({'experts.something_else': torch.randn(2, 3)}, 0, 4)


def test_config_object_resolves_kwargs_and_documents_every_switch():
    import os
    import re
    import subprocess
    import pytest
    from planmoe_b200.utils import config as cf
    cfg = cf.MoEConfig.from_kwargs(gate_type={'type': 'top', 'k': 2}, model_dim=16,
                                   experts={'type': 'ffn', 'count_per_node': 2, 'hidden_size_per_expert': 8},
                                   a2a_ffn_overlap_degree='auto', comm_name='pipe', pad_samples=True)
    layer = cfg.build()
    back = cf.MoEConfig.from_layer(layer)
    assert back.comm_name == 'pipe' and back.a2a_ffn_overlap_degree == 'auto' and back.model_dim == 16
    with pytest.raises(Exception, match='Unrecognized argument'):
        cf.MoEConfig.from_kwargs(model_dim=16, bogus=1)
    with pytest.raises(AssertionError):
        cf.MoEConfig.from_kwargs(model_dim=16, a2a_ffn_overlap_degree=64)
    # every PLANMOE_* switch that the sources read is in the documentation table
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.run(['grep', '-rhoE', r"(environ\.get\(|getenv\()['\"]PLANMOE_[A-Z0-9_]+", os.path.join(root, 'planmoe_b200')],
                         stdout=subprocess.PIPE, text=True).stdout
    used = set(re.findall(r'PLANMOE_[A-Z0-9_]+', out))
    missing = used - set(cf.ENV)
    assert not missing, missing
    assert 'PLANMOE_WAIT_BUDGET_MS' in cf.runtime_env()
