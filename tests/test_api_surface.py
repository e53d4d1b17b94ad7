"""Public API surface: package aliases, facades, launcher command construction, scheduler, the
reference-named native functions, codecs and comm registries on CPU."""

import json
import os
import sys

import pytest
import torch


def test_alias_packages_expose_the_same_modules():
    import planmoe
    import schemoe
    import planmoe_b200
    from schemoe.moe import moe_layer as a
    from planmoe.moe import moe_layer as b
    assert a is b is planmoe_b200.moe.moe_layer
    import planmoe.impls.communicate as c1
    import planmoe_b200.impls.communicate as c2
    assert c1 is c2
    from planmoe import net, system, jit, moe
    for name in ('get_world_size', 'get_world_rank', 'create_groups_from_world', 'barrier', 'simple_all_reduce',
                 'simple_all_to_all', 'simple_split', 'simple_reduce_scatter', 'simple_all_gather', 'all_to_all',
                 'all_to_all_single', 'all_gather', 'zero_gather', 'zero_scatter', 'spatial_split',
                 'reduce_scatter', 'allreduce_forward', 'allreduce_backward', 'TutelDistributedOptimizer'):
        assert hasattr(net, name), name
    for name in ('init_affinity_at_program_beginning', 'init_data_model_parallel', 'cache', 'LocalCache',
                 'get_local_session', 'record_time', 'TUTEL_CUDA_SANDBOX'):
        assert hasattr(system, name), name
    for name in ('moe_layer', 'top_k_routing', 'extract_critical', 'fast_encode', 'fast_decode', 'fast_dispatcher',
                 'fast_cumsum_sub_one'):
        assert hasattr(moe, name), name
    assert callable(jit.create_cuda_kernel)
    for name in ('AllToAllStatus', 'pre_expert_permute', 'post_expert_permute', 'CurrentStreamRelease',
                 'CurrentStreamAcquire', 'NcclStreamRelease', 'NcclStreamAcquire', 'AllToAll2DAsync',
                 'AllToAllScatterAsync', 'AllToAllGatherAsync', 'RestoreBackward', 'PrimAllToAll2D', 'PrimAllToAll',
                 'PrimBwdAllreduce', 'PrimFwdAllreduce', 'PrimReducescatter', 'PrimAllgather', 'PrimSpatialSplit'):
        assert hasattr(c2, name), name
    from planmoe.gates.top import Gate  # noqa: F401
    from planmoe.gates.cosine_top import Gate as G2  # noqa: F401
    from planmoe.experts.ffn import ExpertModule  # noqa: F401
    from planmoe.impls.overlap import a2a_ffn_overlap_forward  # noqa: F401
    import schemoe_custom_kernel as k
    for name in ('compress_operation', 'comm_operation', 'decompress_operation', 'clear_ptr_lst', 'init_nccl',
                 'get_nccl_unique_id', 'get_nccl_unique_id_size', 'invoke', 'inject_source', 'invoke_cpu_fp32',
                 'invoke_cpu_fp64', 'update_sdk_home', 'current_stream_acquire', 'nccl_stream_release'):
        assert hasattr(k, name), name


def test_tutel_ops_cumsum_torch_operator():
    import planmoe_b200.jit_kernels.gating  # noqa: F401  (registers the operator)
    mask = (torch.rand(37, 5) > 0.5).to(torch.int32)
    out = torch.ops.tutel_ops.cumsum(mask)
    assert torch.equal(out, torch.cumsum(mask, dim=0) - 1)


def test_system_cache_and_timer():
    from planmoe_b200 import system
    system.cache().reset()
    system.cache().set('a', 1)
    system.cache().set('b', 2)
    assert system.cache().get('a') == 1 and sorted(system.cache().get()) == [1, 2]
    assert system.record_time(is_cuda=False) > 0
    with pytest.raises(Exception):
        system.LocalCache.reset()
        del system.init_data_model_parallel.__dict__['default_env']
        system.get_local_session()
    system.init_affinity_at_program_beginning()


def test_fifo_pipeline_single_rank_roundtrip():
    import schemoe_custom_kernel as k
    x = torch.relu(torch.randn(4, 8, 32))
    k.clear_ptr_lst()
    parts = []
    for c in x.split(4, dim=1):
        t = k.compress_operation(c.contiguous(), 'int8', 'naive')
        parts.append(k.comm_operation(t))
    outs = [k.decompress_operation(p) for p in parts]
    y = torch.cat(outs, dim=1)
    assert (y - x).abs().max() <= (x.max() - x.min()) / 255 * 0.51 + 1e-6
    k.clear_ptr_lst()
    assert torch.equal(k.decompress_operation(k.comm_operation(k.compress_operation(x, 'nonsense', 'nonsense'))), x)


def test_cpu_sparse_invoke_matches_torch():
    import schemoe_custom_kernel as k
    S, M, E, C = 10, 6, 3, 4
    x = torch.randn(S, M)
    idx = torch.randint(0, E, (S,), dtype=torch.int32)
    loc = torch.zeros(S, dtype=torch.int32)
    cnt = [0] * E
    for t in range(S):
        loc[t] = cnt[int(idx[t])]; cnt[int(idx[t])] += 1
    g = torch.rand(S)
    disp = torch.zeros(E * C, M)
    k.invoke_cpu_fp32([g, idx, loc, x, disp], [S, M, C], 0)
    ref = torch.zeros(E * C, M)
    for t in range(S):
        if loc[t] < C:
            ref[int(idx[t]) * C + int(loc[t])] += g[t] * x[t]
    assert torch.allclose(disp, ref, atol=1e-6)
    back = torch.empty(S, M)
    k.invoke_cpu_fp32([g, idx, loc, back, disp], [S, M, C], 1)
    gg = torch.empty(S)
    k.invoke_cpu_fp32([gg, idx, loc, x, disp], [S, M, C], 2)
    for t in range(S):
        if loc[t] < C:
            row = disp[int(idx[t]) * C + int(loc[t])]
            assert torch.allclose(back[t], g[t] * row, atol=1e-6)
            assert abs(float(gg[t]) - float((row * x[t]).sum())) < 1e-4
        else:
            assert float(back[t].abs().sum()) == 0 and float(gg[t]) == 0


def test_launcher_commands():
    from planmoe_b200.launcher import run, execl
    cmd, env = run.build_command(['-m', 'planmoe_b200.examples.pre_test', '--encode', 'int8'],
                                 {'OMPI_COMM_WORLD_SIZE': '2', 'OMPI_COMM_WORLD_RANK': '1', 'LOCAL_SIZE': '4',
                                  'MASTER_ADDR': 'hostA'})
    assert '--nproc_per_node=4' in cmd and '--nnodes=2' in cmd and '--node_rank=1' in cmd
    assert '--master_addr=hostA' in cmd and cmd[-3:] == ['planmoe_b200.examples.pre_test', '--encode', 'int8']
    assert 'planmoe_b200.launcher.execl' in cmd and env['LOCAL_SIZE'] == '4'
    cmd, env = execl.build_command(['python', 'x.py'], {'LOCAL_RANK': '3', 'TUTEL_CUDA_SANDBOX': '2', 'LOCAL_SIZE': '8'})
    assert env['CUDA_VISIBLE_DEVICES'] == '3' and cmd[-2:] == ['python', 'x.py']


def _two_rank_scheduler(scheduler, monkeypatch, key, **kw):
    """A scheduler that believes it has a peer; the collectives over the group are identities."""
    sch = scheduler.AdaptiveScheduler(key, **kw)
    monkeypatch.setattr(sch, '_world', lambda: 2)
    monkeypatch.setattr(sch, '_bcast_obj', lambda obj: obj)
    monkeypatch.setattr(sch, '_max_over_ranks', lambda values, device: list(values))
    return sch


def test_adaptive_scheduler_single_rank_needs_no_measurement():
    from planmoe_b200.parallel import scheduler
    sch = scheduler.AdaptiveScheduler('single', degrees=(1, 2, 4), use_cache=False)
    calls = []
    assert sch.resolve(lambda d, c: calls.append(d), torch.device('cpu')) == (1, None)
    assert not calls and sch.report['source'] == 'single rank'


def test_adaptive_scheduler_is_stable_under_noise_and_caches(tmp_path, monkeypatch):
    """Noisy synthetic timings: the choice is the same for every noise seed; near-ties resolve to fewer chunks."""
    import random
    import time
    from planmoe_b200.parallel import scheduler
    monkeypatch.setenv('PLANMOE_PLAN_CACHE', str(tmp_path / 'plans.json'))
    fake = [0.0]
    monkeypatch.setattr(time, 'perf_counter', lambda: fake[0])

    def decide(cost, noise, seed, key):
        rng = random.Random(seed)
        sch = _two_rank_scheduler(scheduler, monkeypatch, key, degrees=(1, 2, 4, 8), use_cache=False)

        def run(d, comm):
            fake[0] += cost[d] * 1e-3 * (1.0 + rng.uniform(-noise, noise))
            if rng.random() < 0.1:
                fake[0] += cost[d] * 1e-3          # an occasional outlier twice as long
        return sch.resolve(run, torch.device('cpu'))[0]

    near_tie = {1: 1.00, 2: 0.99, 4: 1.01, 8: 1.20}
    assert {decide(near_tie, 0.02, s, 'a%d' % s) for s in range(40)} == {1}
    clear = {1: 1.30, 2: 1.12, 4: 1.00, 8: 1.20}
    assert {decide(clear, 0.02, s, 'b%d' % s) for s in range(40)} == {4}

    sch = _two_rank_scheduler(scheduler, monkeypatch, 'k1', degrees=(1, 2, 4))
    assert sch.resolve(lambda d, c: fake.__setitem__(0, fake[0] + clear[d] * 1e-3), torch.device('cpu'))[0] == 4
    assert json.load(open(tmp_path / 'plans.json'))['k1']['degree'] == 4
    again = _two_rank_scheduler(scheduler, monkeypatch, 'k1', degrees=(1, 2, 4))
    calls = []
    assert again.resolve(lambda d, c: calls.append(d), torch.device('cpu'))[0] == 4
    assert not calls and again.report['source'] == 'cache'


def test_adaptive_scheduler_picks_the_comm_algorithm_too(monkeypatch):
    import time
    from planmoe_b200.parallel import scheduler
    fake = [0.0]
    monkeypatch.setattr(time, 'perf_counter', lambda: fake[0])
    sch = _two_rank_scheduler(scheduler, monkeypatch, 'c', degrees=(1, 2), comms=('naive', 'pipe', 'hetu'),
                              use_cache=False)
    cost = {('naive', 1): 1.0, ('naive', 2): 0.9, ('pipe', 1): 1.0, ('pipe', 2): 0.8, ('hetu', 1): 2.0, ('hetu', 2): 1.9}
    assert sch.resolve(lambda d, c: fake.__setitem__(0, fake[0] + cost[(c, d)] * 1e-3), torch.device('cpu')) == (2, 'pipe')
    assert set(sch.report['ms']) == {'1/naive', '2/naive', '1/pipe', '2/pipe', '1/hetu', '2/hetu'}


def test_layer_with_auto_degree_runs_on_cpu(tmp_path, monkeypatch):
    from planmoe_b200 import moe
    monkeypatch.setenv('PLANMOE_PLAN_CACHE', str(tmp_path / 'plans.json'))
    layer = moe.moe_layer({'type': 'top', 'k': 2}, 32, experts={'type': 'ffn', 'count_per_node': 2,
                                                            'hidden_size_per_expert': 32},
                          a2a_ffn_overlap_degree='auto')
    x = torch.randn(64, 32)
    ys = [layer(x) for _ in range(3)]
    assert layer._scheduler.frozen == 1          # one rank: no calibration, degree 1
    assert torch.allclose(ys[0], ys[-1], atol=1e-5)


def test_comm_and_codec_registries():
    from planmoe_b200.parallel import codecs, comms
    assert isinstance(codecs.get_compressor('bogus'), codecs.NoCompressor)
    assert isinstance(comms.get_comm('bogus'), comms.NaiveComm)
    for name in ('naive', 'pipe', 'dd', 'hetu', 'nccl'):
        c = comms.get_comm(name)
        t = torch.arange(6.)
        assert torch.equal(c.all_to_all(t), t)           # a world of one rank is the identity

    class Half(codecs.AbstractCompressor):
        name = 'half'

        def compress(self, t, world_size=1):
            return codecs.Packed([t.half()], t.dtype)

        def decompress(self, packed):
            return packed.wires[0].to(packed.meta)
    codecs.register_compressor('half', Half)
    from planmoe_b200.impls.overlap import ChunkHandle
    x = torch.randn(4, 4)
    assert torch.allclose(ChunkHandle('half', 'naive', None).launch(x).finish(), x, atol=1e-2)


def test_pre_test_example_runs_on_cpu(tmp_path):
    from planmoe_b200.examples import pre_test
    mean, err = pre_test.main(['--device', 'cpu', '--dtype', 'float32', '--batch_size', '2', '--num_tokens', '16',
                               '--model_dim', '32', '--hidden_size', '32', '--num_steps', '3',
                               '--a2a_ffn_overlap_degree', '2', '--log', str(tmp_path / 't.log')])
    assert err == 0.0 and mean > 0
    mean, _ = pre_test.main(['--device', 'cpu', '--dtype', 'float32', '--batch_size', '2', '--num_tokens', '16',
                             '--model_dim', '32', '--hidden_size', '32', '--num_steps', '2', '--layer',
                             '--log', str(tmp_path / 't.log')])
    assert mean > 0


def test_cpp_extension_point_registries():
    """Comm / codec objects registered from C++ are reachable by name from the Python layer."""
    from planmoe_b200.ops import native
    from planmoe_b200.parallel import codecs, comms
    lib = native.lib()
    assert 'native_flat' in lib.native_comm_names() and 'native_copy' in lib.native_compressor_names()
    x = torch.randn(4, 6)
    c = comms.get_comm('native_flat')
    assert isinstance(c, comms.NativeComm) and torch.equal(c.all_to_all(x), x)
    k = codecs.get_compressor('native_copy')
    assert isinstance(k, codecs.NativeCompressor)
    assert torch.equal(k.decompress(k.compress(x, 2)), x)


def test_integration_helpers():
    import argparse
    from types import SimpleNamespace
    from planmoe_b200.examples.megatron import planmoe_megatron as pm
    from planmoe_b200.examples.fairseq_moe import planmoe_fairseq as pf
    args = pm.add_planmoe_args(argparse.ArgumentParser()).parse_args(
        ['--schemoe', '--schemoe-overlap-degree', '2', '--schemoe-compress-name', 'int8'])
    assert args.schemoe and args.schemoe_comm_name == 'naive'
    cfg = SimpleNamespace(hidden_size=32, ffn_hidden_size=64, num_moe_experts=4, expert_model_parallel_size=1,
                          moe_router_topk=2, moe_expert_capacity_factor=2.0)
    layer = pm.maybe_replace_mlp(SimpleNamespace(mlp=None), cfg, args)
    out, bias = layer.mlp(torch.randn(2, 8, 32))
    assert out.shape == (2, 8, 32) and bias is None
    assert all(p.allreduce is False for p in layer.mlp.moe.experts.parameters())
    os.environ['MOE'] = '2'
    os.environ['L_AUX_WT'] = '0.01'
    try:
        assert pf.build_ffn(0, 16, 32) is None
        moe = pf.build_ffn(1, 16, 32)
        moe.train()
        y = pf.ffn_forward(moe, torch.randn(6, 16, requires_grad=True))
        total = pf.add_aux_loss(torch.tensor(1.0), sample_size=6)
        assert y.shape == (6, 16) and float(total) > 1.0
    finally:
        os.environ.pop('MOE')
        os.environ.pop('L_AUX_WT')
    p = torch.nn.Parameter(torch.ones(3))
    p.grad = torch.tensor([1.0, float('inf'), float('nan')])
    os.environ['NO_OVERFLOW'] = '1'
    try:
        pf.sanitize_grads([p])
    finally:
        os.environ.pop('NO_OVERFLOW')
    assert p.grad.tolist() == [1.0, 0.0, 0.0]


def test_grid_of_rows_and_columns():
    from planmoe_b200.impls.communicate import grid_of
    g, m, d, r, rows, cols = grid_of(8, 5, 2)
    assert (g, m, d, r) == (2, 4, 1, 1)
    assert rows == [[0, 1, 2, 3], [4, 5, 6, 7]] and cols == [[0, 4], [1, 5], [2, 6], [3, 7]]
    assert 5 in rows[d] and 5 in cols[r]
    g, m, d, r, rows, cols = grid_of(8, 3, -2)            # model groups of two ranks
    assert (g, m, d, r) == (4, 2, 1, 1) and rows[1] == [2, 3] and cols[1] == [1, 3, 5, 7]
    assert grid_of(1, 0, 1)[:4] == (1, 1, 0, 0)
    import pytest
    with pytest.raises(AssertionError):
        grid_of(6, 0, 4)
