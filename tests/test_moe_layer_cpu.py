"""CPU single-process MoE layer against the dense per-token oracle (fp32, W = 1, identity
all-to-all, no compression): outputs, input grads and every parameter grad."""

import pytest
import torch
import torch.nn.functional as F

from planmoe_b200 import moe
from oracle import dense_moe_reference


def _build(E=8, M=256, H=512, k=2, cf=1.0, **kw):
    torch.manual_seed(0)
    layer = moe.moe_layer(
        gate_type={'type': 'top', 'k': k, 'capacity_factor': cf},
        model_dim=M,
        experts={'type': 'ffn', 'count_per_node': E, 'hidden_size_per_expert': H,
                 'activation_fn': lambda x: F.relu(x)},
        seeds=(1, 2, 3), **kw)
    return layer


@pytest.mark.parametrize("degree", [1, 2])
@pytest.mark.parametrize("postscore", [True, False])
def test_config1_matches_dense_oracle(degree, postscore):
    layer = _build(is_postscore=postscore, a2a_ffn_overlap_degree=degree)
    torch.manual_seed(0)
    x = torch.randn(4, 128, 256, requires_grad=True)
    y = layer(x)
    assert y.shape == x.shape and y.dtype == x.dtype
    loss = (y * torch.linspace(-1, 1, y.numel()).view_as(y)).sum() + y.l_aux
    loss.backward()

    xr = x.detach().clone().reshape(-1, 256).requires_grad_(True)
    ex = layer.experts
    params = [layer.gates[0].wg.weight, ex.batched_fc1_w, ex.batched_fc1_bias, ex.batched_fc2_w, ex.batched_fc2_bias]
    refp = [p.detach().clone().requires_grad_(True) for p in params]
    yr, l_aux = dense_moe_reference(xr, *refp, top_k=2, capacity_factor=1.0, alignment=4 * degree,
                                    is_postscore=postscore)
    lr = (yr.view_as(y) * torch.linspace(-1, 1, y.numel()).view_as(y)).sum() + l_aux
    lr.backward()

    assert torch.allclose(y.reshape(-1, 256), yr, atol=2e-5, rtol=1e-4)
    assert torch.allclose(y.l_aux, l_aux, atol=1e-6)
    assert torch.allclose(x.grad.reshape(-1, 256), xr.grad, atol=2e-4, rtol=1e-3)
    for p, r in zip(params, refp):
        assert torch.allclose(p.grad, r.grad, atol=2e-4, rtol=1e-3), (p.shape, (p.grad - r.grad).abs().max())


def test_state_dict_keys_and_shapes():
    layer = _build(E=4, M=64, H=96)
    sd = layer.state_dict()
    assert set(sd) == {'gates.0.wg.weight', 'experts.batched_fc1_w', 'experts.batched_fc2_w',
                       'experts.batched_fc1_bias', 'experts.batched_fc2_bias'}
    assert sd['gates.0.wg.weight'].shape == (4, 64)
    assert sd['experts.batched_fc1_w'].shape == (4, 64, 96)
    assert sd['experts.batched_fc2_w'].shape == (4, 96, 64)
    assert sd['experts.batched_fc1_bias'].shape == (4, 96)
    assert sd['experts.batched_fc2_bias'].shape == (4, 64)
    other = _build(E=4, M=64, H=96)
    other.load_state_dict(sd)
    for p in layer.experts.parameters():
        assert getattr(p, '_tutel_expert', False)


def test_seeded_init_reproduces_linear_init_order():
    """Expert weights come from nn.Linear default init, expert by expert, under seeds[1]."""
    layer = _build(E=2, M=32, H=48)
    torch.manual_seed(2)
    for e in range(2):
        fc1 = torch.nn.Linear(32, 48)
        fc2 = torch.nn.Linear(48, 32)
        assert torch.equal(layer.experts.batched_fc1_w[e], fc1.weight.t())
        assert torch.equal(layer.experts.batched_fc2_bias[e], fc2.bias)


def test_constructor_contract():
    with pytest.raises(Exception, match='Unrecognized argument'):
        _build(bogus=1)
    with pytest.raises(AssertionError):
        moe.moe_layer({'type': 'top', 'k': 1}, 33, experts={'type': 'ffn', 'count_per_node': 1,
                                                           'hidden_size_per_expert': 8})
    layer = moe.moe_layer('Top2Gate', 32, experts={'type': 'ffn', 'count_per_node': 2,
                                                  'hidden_size_per_expert': 16})
    assert layer.gates[0].top_k == 2
    assert len(list(layer.get_parameter_iterator('gate'))) == 1
    assert len(list(layer.get_parameter_iterator('local_experts'))) == 4
    with pytest.raises(Exception):
        layer.get_parameter_iterator('nope')
    assert 'Top-K(s)' in layer.extra_repr()


def test_forward_overrides_and_result_func():
    layer = _build(E=4, M=32, H=32, result_func=lambda y: y * 2)
    x = torch.randn(16, 32)
    y2 = layer(x, top_k=1, capacity_factor=2.0)
    layer.result_func = None
    y1 = layer(x, top_k=1, capacity_factor=2.0)
    assert torch.allclose(y2, y1 * 2)
    yd = layer(x, capacity_factor=0.0)          # dynamic capacity: nothing dropped
    yl = layer(x, capacity_factor=100.0)
    assert torch.allclose(yd, yl, atol=1e-6)


def test_cosine_gate_and_custom_expert_and_multi_gate():
    class Twice(torch.nn.Module):
        def update(self, ctx):
            self.scale = torch.nn.Parameter(torch.full((ctx.num_local_experts, 1, 1), 2.0))

        def forward(self, x, ctx):
            return x * self.scale

    layer = moe.moe_layer(
        gate_type=[{'type': 'cosine_top', 'k': 1, 'proj_dim': 16}, {'type': 'top', 'k': 2}],
        model_dim=32, experts={'type': 'custom', 'module': Twice(), 'count_per_node': 3})
    assert 'gates.0.sim_matrix' in layer.state_dict() and 'gates.1.wg.weight' in layer.state_dict()
    x = torch.randn(12, 32)
    y = layer(x, gate_index=0, capacity_factor=4.0)
    g = F.softmax(layer.gates[0](x), dim=1).max(dim=1).values
    assert torch.allclose(y, 2 * x * g[:, None], atol=1e-5)
    layer(x, gate_index=1).sum().backward()


def test_batch_prioritized_and_load_importance_loss_run():
    layer = _build(E=4, M=32, H=32, batch_prioritized_routing=True, is_gshard_loss=False)
    layer.gates[0].gate_noise = 1.0
    x = torch.randn(64, 32, requires_grad=True)
    y = layer(x)
    (y.sum() + y.l_aux).backward()
    assert torch.isfinite(x.grad).all() and torch.isfinite(y.l_aux)


@pytest.mark.parametrize("E,k,cf,S", [(1, 1, 1.0, 37), (2, 1, 0.5, 64), (4, 4, 1.0, 50), (8, 2, 0.25, 96), (3, 2, 2.0, 10)])
def test_edge_shapes_match_dense_oracle(E, k, cf, S):
    """One expert, top-1, top-k = all experts, tight capacity (many dropped tokens), odd token counts."""
    M, H = 32, 48
    layer = _build(E=E, M=M, H=H, k=k, cf=cf)
    torch.manual_seed(3)
    x = torch.randn(S, M, requires_grad=True)
    y = layer(x)
    (y.sum() + y.l_aux).backward()
    ex = layer.experts
    params = [layer.gates[0].wg.weight, ex.batched_fc1_w, ex.batched_fc1_bias, ex.batched_fc2_w, ex.batched_fc2_bias]
    refp = [p.detach().clone().requires_grad_(True) for p in params]
    xr = x.detach().clone().requires_grad_(True)
    yr, l_aux = dense_moe_reference(xr, *refp, top_k=k, capacity_factor=cf, alignment=4)
    (yr.sum() + l_aux).backward()
    assert torch.allclose(y, yr, atol=2e-5, rtol=1e-4)
    assert torch.allclose(x.grad, xr.grad, atol=2e-4, rtol=1e-3)
    for p, r in zip(params, refp):
        assert torch.allclose(p.grad, r.grad, atol=2e-4, rtol=1e-3)


def test_all_tokens_to_one_expert_and_an_idle_expert():
    """A gate that sends every token to expert 0: the other experts see no token (zero gradients), tokens
    beyond the capacity are dropped, and the layer still matches the oracle."""
    E, M, H, S = 4, 16, 24, 40
    layer = _build(E=E, M=M, H=H, k=1, cf=1.0)
    with torch.no_grad():
        layer.gates[0].wg.weight.zero_()
        layer.gates[0].wg.weight[0].fill_(5.0)
    x = (torch.rand(S, M) + 0.5).requires_grad_(True)          # positive inputs: expert 0 always wins
    y = layer(x)
    y.sum().backward()
    ex = layer.experts
    assert ex.batched_fc1_w.grad[1:].abs().max() == 0 and ex.batched_fc2_w.grad[1:].abs().max() == 0
    cap = layer.last_stats['capacity']
    assert (y.abs().sum(dim=1) > 0).sum() == min(cap, S)       # tokens beyond the capacity produce zeros
    params = [layer.gates[0].wg.weight, ex.batched_fc1_w, ex.batched_fc1_bias, ex.batched_fc2_w, ex.batched_fc2_bias]
    yr, _ = dense_moe_reference(x.detach(), *[p.detach() for p in params], top_k=1, capacity_factor=1.0, alignment=4)
    assert torch.allclose(y, yr, atol=2e-5, rtol=1e-4)
