"""parted: format parser, plan search on an MLP graph, code generation, and execution of generated
programs (1 rank in-process launch; 2 Gloo ranks through torchrun) with equal digests across plans."""

import json
import os
import subprocess
import sys

import pytest


@pytest.fixture()
def spmdx(monkeypatch):
    for k in ('STRICT_FMT', 'PTYPE', 'CONFIG'):
        monkeypatch.delenv(k, raising=False)
    from planmoe_b200.parted import spmdx as S
    S.init('torch', reset=True)
    return S


def _mlp(S, B=8, M=16, H=32):
    x = S.Tensor([B, M], 'float32')
    w1 = S.Tensor([M, H], 'float32', is_param=True)
    w2 = S.Tensor([H, M], 'float32', is_param=True)

    def Matmul(a, b, ir):
        return S.Custom(ir, 'torch.matmul(%s, %s)' % (a, b))

    def Relu(a):
        return S.Custom('bh = bh', 'torch.relu(%s)' % a)
    h = Relu(Matmul(x, w1, 'bh += bm, mh'))
    return Matmul(h, w2, 'bm += bh, hm')


def test_parser_and_shapes(spmdx):
    p = spmdx.Parser('b(hd) += bm, m(hd)')
    assert p.reduce_type == '+' and p.get_reduce_axes() == {'m'}
    assert p.left.id2ax == ['b', ['h', 'd']]
    dims, parted = p.emit_dims_by_name('h')
    assert dims == {0: -1, 1: 1} and parted == 1
    with pytest.raises(NotImplementedError):
        p.emit_dims_by_name('d')
    y = _mlp(spmdx)
    assert y.shape == [8, 16] and y.flops == 2 * 8 * 16 * 32


def test_plan_search_finds_tensor_and_data_parallel_plans(spmdx):
    y = _mlp(spmdx)
    cfg = y.autotune(total_nodes=2, device_type='cpu', run_mode='train')
    plan = cfg.config['b']
    assert cfg.config['v'] == '0.1' and set(plan) >= {y.name}
    kwargs, results = spmdx.optimize(y, total_nodes=2, device_type='cpu')
    states = {dim: sol for dim, sol in results if sol is not None}
    assert -1 in states and 0 in states
    prims = {v[1].split(':')[0] for sol in states.values() for v in sol[1].values() if v[1]}
    assert prims & {'FAR', 'RS', 'BAR', 'AG', 'SPLIT', 'A2A', 'ZERO'}


def test_config_roundtrip_and_data_parallel_config(spmdx, tmp_path):
    y = _mlp(spmdx)
    cfg = y.get_data_parallel_config(total_nodes=2, device_type='cpu')
    path = tmp_path / 'plan.json'
    cfg.save(str(path))
    again = spmdx.Config.load_from_file(str(path))
    assert json.loads(str(again)) == cfg.config
    with pytest.raises(Exception):
        spmdx.Config({'v': '9.9'})


def test_generated_program_runs_single_rank(spmdx, tmp_path):
    y = _mlp(spmdx)
    cfg = y.autotune(total_nodes=1, device_type='cpu', run_mode='train')
    prog = y.compile(cfg)
    assert 'class DistModel' in prog.code
    out = prog.execute()
    assert out.get('name') == y.name and out['step_time'] > 0


def test_two_rank_plans_give_the_same_digest(spmdx):
    y = _mlp(spmdx)
    _, results = spmdx.optimize(y, total_nodes=2, device_type='cpu', run_mode='infer')
    digests = []
    for dim, sol in results:
        if sol is None:
            continue
        prog = y.compile(sol[1], total_nodes=2, device_type='cpu', run_mode='infer')
        out = prog.execute()
        assert out.get('step_time', 0) > 0, prog.code
        digests.append(out['digest'])
    assert len(digests) >= 2
    assert all(abs(d - digests[0]) < 1e-5 for d in digests), digests
