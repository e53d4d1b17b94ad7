"""The fused sm_100a MoE path on one GPU against a plain PyTorch fp32 reference of the layer."""

import os

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu
os.environ.setdefault('PLANMOE_WAIT_BUDGET_MS', '3000')

from oracle import dense_moe_reference  # noqa: E402


def _layer(E, M, H, k, cf, act='gelu', **kw):
    from planmoe_b200 import moe
    torch.manual_seed(0)
    layer = moe.moe_layer(gate_type={'type': 'top', 'k': k, 'capacity_factor': cf, 'fp32_gate': True},
                          model_dim=M,
                          experts={'type': 'ffn', 'count_per_node': E, 'hidden_size_per_expert': H,
                                   'activation_fn': act},
                          seeds=(1, 2, 3), **kw)
    return layer.cuda().to(torch.bfloat16)


@pytest.mark.parametrize("degree", [1, 2])
@pytest.mark.parametrize("postscore", [True, False])
@pytest.mark.parametrize("fuse_send", [0, 1])
def test_fused_layer_matches_fp32_reference(degree, postscore, fuse_send, monkeypatch):
    """``fuse_send`` = 1 runs the dispatch send inside the flag-gated GEMM launch (copy warps)."""
    monkeypatch.setenv('PLANMOE_FUSE_SEND', str(fuse_send))
    E, M, H, k, cf = 4, 256, 512, 2, 1.0
    layer = _layer(E, M, H, k, cf, is_postscore=postscore, a2a_ffn_overlap_degree=degree)
    layer.gates[0].wg.float()
    torch.manual_seed(0)
    x = torch.randn(2048, M, device='cuda').to(torch.bfloat16).requires_grad_(True)
    y = layer(x)
    assert layer.last_stats['path'] == 'fused'
    w = torch.linspace(-1, 1, y.numel(), device='cuda').view_as(y)
    ((y.float() * w).sum() + y.l_aux.float()).backward()
    from planmoe_b200.parallel import transport
    transport.get_transport(layer.group).check()

    ex = layer.experts
    params = [layer.gates[0].wg.weight, ex.batched_fc1_w, ex.batched_fc1_bias, ex.batched_fc2_w, ex.batched_fc2_bias]
    refp = [p.detach().float().cpu().requires_grad_(True) for p in params]
    xr = x.detach().float().cpu().requires_grad_(True)
    yr, l_aux = dense_moe_reference(xr, *refp, top_k=k, capacity_factor=cf, act=F.gelu,
                                    alignment=4 * degree, is_postscore=postscore)
    ((yr * w.cpu()).sum() + l_aux).backward()

    def close(a, b, tol):
        a, b = a.float().cpu(), b.float()
        return ((a - b).abs().max() / (b.abs().max() + 1e-6)).item() < tol

    assert close(y, yr, 3e-2)
    assert abs(y.l_aux.item() - l_aux.item()) < 1e-3
    assert close(x.grad, xr.grad, 4e-2)
    for p, r in zip(params, refp):
        assert close(p.grad, r.grad, 5e-2), p.shape


@pytest.mark.parametrize("degree", [1, 2])
def test_fused_layer_int8_wire_matches_fp32_reference(degree):
    """compress_name='int8' on the fused path: rows are quantised before the send, de-quantised in front of the
    GEMMs by the de-quantiser warps, pushed back as int8 by the GEMM epilogues and de-quantised by the gathers."""
    E, M, H, k, cf = 4, 256, 512, 2, 1.0
    layer = _layer(E, M, H, k, cf, a2a_ffn_overlap_degree=degree, compress_name='int8')
    layer.gates[0].wg.float()
    torch.manual_seed(0)
    x = torch.randn(2048, M, device='cuda').to(torch.bfloat16).requires_grad_(True)
    y = layer(x)
    assert layer.last_stats['path'] == 'fused' and layer.last_stats['wire'] == 'int8'
    w = torch.linspace(-1, 1, y.numel(), device='cuda').view_as(y)
    ((y.float() * w).sum() + y.l_aux.float()).backward()
    from planmoe_b200.parallel import transport
    transport.get_transport(layer.group).check()

    ex = layer.experts
    params = [layer.gates[0].wg.weight, ex.batched_fc1_w, ex.batched_fc1_bias, ex.batched_fc2_w, ex.batched_fc2_bias]
    refp = [p.detach().float().cpu().requires_grad_(True) for p in params]
    xr = x.detach().float().cpu().requires_grad_(True)
    yr, l_aux = dense_moe_reference(xr, *refp, top_k=k, capacity_factor=cf, act=F.gelu, alignment=4 * degree)
    ((yr * w.cpu()).sum() + l_aux).backward()

    def err(a, b):
        a, b = a.float().cpu(), b.float()
        return ((a - b).abs().max() / (b.abs().max() + 1e-6)).item()

    assert err(y, yr) < 6e-2, err(y, yr)
    assert err(x.grad, xr.grad) < 0.15, err(x.grad, xr.grad)
    for p, r in zip(params, refp):
        assert err(p.grad, r.grad) < 0.15, (p.shape, err(p.grad, r.grad))
    # and it really differs from the bf16 wire (the quantisation is not a no-op)
    layer2 = _layer(E, M, H, k, cf, a2a_ffn_overlap_degree=degree)
    layer2.load_state_dict(layer.state_dict())
    layer2.gates[0].wg.float()
    with torch.no_grad():
        y2 = layer2(x.detach())
    assert not torch.equal(y2, y.detach())


@pytest.mark.parametrize("variant", ['cf_negative', 'cf_zero_dynamic', 'batch_prio', 'load_importance', 'fairseq_like'])
def test_routing_variants_stay_on_the_fused_path(variant, monkeypatch):
    """Dynamic / bounded capacity, batch-prioritised routing and the load-importance loss run on the fused kernels
    and agree with the generic path (ATen routing of ``extract_critical``, torch.matmul experts)."""
    E, M, H, k = 4, 256, 256, 2
    kw, cf = {}, 1.0
    if variant == 'cf_negative':
        cf = -1.5
    elif variant == 'cf_zero_dynamic':
        cf = 0.0
    elif variant == 'batch_prio':
        kw['batch_prioritized_routing'] = True
        cf = 0.5                                   # tight capacity: which tokens are dropped depends on the order
    elif variant == 'load_importance':
        kw['is_gshard_loss'] = False
    elif variant == 'fairseq_like':
        E, cf = 1, 0.0                             # one expert per GPU, dynamic capacity (the fairseq integration)
    layer = _layer(E, M, H, k, cf, **kw)
    layer.gates[0].wg.float()
    if variant == 'load_importance':
        layer.gates[0].gate_noise = 1.0            # the loss's load term needs a noise scale; eval mode adds no noise
        layer.eval()
    torch.manual_seed(3)
    x0 = torch.randn(1536, M, device='cuda').to(torch.bfloat16)
    w = torch.linspace(-1, 1, x0.numel(), device='cuda').view_as(x0)

    def run(fused):
        monkeypatch.setenv('PLANMOE_FUSED', '1' if fused else '0')
        x = x0.clone().requires_grad_(True)
        y = layer(x)
        assert layer.last_stats['path'] == ('fused' if fused else 'generic')
        ((y.float() * w).sum() + y.l_aux.float()).backward()
        g = layer.gates[0].wg.weight.grad.clone()
        layer.zero_grad()
        return y.detach().float(), float(y.l_aux), x.grad.float(), g, layer.last_stats['capacity']

    yf, lf, gxf, gwf, cap_f = run(True)
    from planmoe_b200.parallel import transport
    transport.get_transport(layer.group).check()
    yg, lg, gxg, gwg, cap_g = run(False)
    if variant in ('cf_zero_dynamic', 'fairseq_like'):
        assert cap_f >= cap_g                      # the fused path rounds the dynamic capacity up, never down
    close = lambda a, b, tol: ((a - b).abs().max() / (b.abs().max() + 1e-6)).item() < tol   # noqa: E731
    assert close(yf, yg, 3e-2)
    assert abs(lf - lg) < 1e-3 * max(1.0, abs(lg)), (lf, lg)
    assert close(gxf, gxg, 4e-2)
    assert close(gwf.float(), gwg.float(), 5e-2)


def test_importance_order_kernel_matches_a_sort():
    from planmoe_b200.ops import native
    lib = native.lib()
    torch.manual_seed(0)
    logits = torch.randn(3000, 16, device='cuda')
    logits[100] = logits[7]                         # a tie: the lower token index goes first
    rank, perm = lib.importance_order(logits)
    key = F.softmax(logits.double(), dim=1).max(dim=1).values
    along = key[perm.long()]
    assert bool((along[:-1] - along[1:] >= -1e-6).all())          # best top score first
    pos = rank.tolist()
    assert pos[7] + 1 == pos[100]                                   # equal keys: token order
    assert rank[perm.long()].tolist() == list(range(3000))          # rank and perm are inverse permutations


def test_debug_guards_and_poisoned_receive_buffers(monkeypatch):
    """PLANMOE_DEBUG_GUARDS=1: heap blocks sit between canary bands and receive buffers start as NaN.  A correct
    layer step leaves the canaries intact and produces finite numbers (every slot it reads was written); a write
    just past a block, made from the host side through a view of the heap, is reported by check()."""
    from planmoe_b200.parallel import transport
    monkeypatch.setenv('PLANMOE_DEBUG_GUARDS', '1')
    layer = _layer(2, 256, 256, 2, 1.0)
    x = torch.randn(1024, 256, device='cuda').to(torch.bfloat16).requires_grad_(True)
    for _ in range(3):
        y = layer(x)
        y.float().sum().backward()
    tr = transport.get_transport(layer.group)
    tr.check()
    assert torch.isfinite(y.float()).all() and torch.isfinite(x.grad.float()).all()
    blk = tr.alloc(4096)
    from planmoe_b200.ops import native
    past = native.lib().tensor_from_ptr(blk.local_ptr + blk.nbytes, 16, torch.cuda.current_device())
    past.fill_(0)                                            # 16 bytes of the upper guard band
    with pytest.raises(transport.TransportError, match='guard band'):
        tr.check()
    past.fill_(0xA5)
    tr.check()


def test_fused_layer_is_bit_reproducible_and_reuses_buffers():
    layer = _layer(2, 256, 256, 2, 1.0)
    x = torch.randn(1024, 256, device='cuda').to(torch.bfloat16)
    outs = []
    for _ in range(4):
        xi = x.clone().requires_grad_(True)
        y = layer(xi)
        y.float().sum().backward()
        outs.append((y.detach().clone(), xi.grad.clone()))
    for y, g in outs[1:]:
        assert torch.equal(y, outs[0][0]) and torch.equal(g, outs[0][1])
    rings = layer._fused.sets
    assert all(len(r) <= 2 for r in rings.values())
    with torch.no_grad():
        y = layer(x)
    assert torch.equal(y, outs[0][0])


def test_fused_layer_survives_degree_changes():
    """The adaptive scheduler switches the pipeline degree between steps of one layer."""
    layer = _layer(2, 256, 256, 2, 1.0)
    x = torch.randn(1024, 256, device='cuda').to(torch.bfloat16)
    outs = []
    from planmoe_b200.parallel import transport
    for d in (1, 2, 4, 1, 4, 2):
        xi = x.clone().requires_grad_(True)
        y = layer(xi, a2a_ffn_overlap_degree=d)
        y.float().sum().backward()
        transport.get_transport(layer.group).check()
        outs.append(y.detach().clone())
    for y in outs[1:]:
        assert torch.equal(y, outs[0])


@pytest.mark.parametrize('split', [False, True])
def test_fused_layer_replays_under_cuda_graph(split):
    """Two training steps (forward + backward + SGD) captured in one CUDA graph, or in one graph each, and replayed
    give the same parameters as the same number of eager steps."""
    from planmoe_b200.parallel import transport
    from planmoe_b200.utils.graphs import GraphedSteps

    def make():
        layer = _layer(2, 256, 256, 2, 1.0)
        opt = torch.optim.SGD(layer.parameters(), lr=1e-2)
        return layer, opt

    torch.manual_seed(0)
    x = torch.randn(1024, 256, device='cuda').to(torch.bfloat16)

    def one_step(layer, opt):
        opt.zero_grad(set_to_none=True)
        y = layer(x)
        loss = y.float().pow(2).mean() + 0.01 * y.l_aux.float()
        loss.backward()
        opt.step()
        return loss.detach().reshape(1)

    warm, unroll, replays = 2, 2, 3
    layer_e, opt_e = make()
    for _ in range(warm * unroll + replays * unroll):     # the capture pass itself executes nothing
        one_step(layer_e, opt_e)
    layer_g, opt_g = make()
    g = GraphedSteps(lambda: one_step(layer_g, opt_g), unroll=unroll, warmup=warm, split=split)
    for _ in range(replays):
        outs = [g.replay_one(0), g.replay_one(1)] if split else g.replay()
    torch.cuda.synchronize()
    transport.get_transport(layer_g.group).check()
    assert torch.isfinite(outs[-1]).all()
    for pe, pg in zip(layer_e.parameters(), layer_g.parameters()):
        assert torch.equal(pe, pg), pe.shape


def test_generic_cuda_path_matches_fused():
    """Same layer through the generic pipeline (torch.matmul experts) and through the fused path."""
    layer = _layer(4, 256, 256, 2, 2.0, act='relu')
    x = torch.randn(512, 256, device='cuda').to(torch.bfloat16)
    with torch.no_grad():
        y_fused = layer(x)
        os.environ['PLANMOE_FUSED'] = '0'
        os.environ['PLANMOE_GEMM'] = 'cublas'
        try:
            y_gen = layer(x)
        finally:
            os.environ.pop('PLANMOE_FUSED'); os.environ.pop('PLANMOE_GEMM')
    assert layer.last_stats is not None
    assert ((y_fused.float() - y_gen.float()).abs().max() / y_gen.float().abs().max()).item() < 3e-2


def test_plans_outside_the_fused_limits_take_the_generic_path():
    """top-8 (the fused gate stops at top-4) must not reach the fused kernels: the layer answers through the generic
    path; a pipeline degree above the flag table's 32 chunks is refused instead of overrunning the flags."""
    from planmoe_b200.parallel import transport
    layer = _layer(16, 256, 256, 8, 1.0, act='relu')
    x = torch.randn(512, 256, device='cuda').to(torch.bfloat16).requires_grad_(True)
    y = layer(x)
    assert layer.last_stats['path'] == 'generic' and torch.isfinite(y.float()).all()
    y.float().sum().backward()
    assert torch.isfinite(x.grad.float()).all()
    # the same layer with a per-call top-2 override is inside the limits again
    y2 = layer(x, top_k=2)
    assert layer.last_stats['path'] == 'fused' and torch.isfinite(y2.float()).all()
    # a degree above the 32 chunks that both the flag tables and AllToAllStatus.max_num_split allow is refused
    # before any kernel runs (the reference asserts the same limit, PlanMoE/impls/overlap.py:49-50)
    layer2 = _layer(2, 256, 256, 2, 1.0)
    xb = torch.randn(4096, 256, device='cuda').to(torch.bfloat16)
    with torch.no_grad():
        with pytest.raises(AssertionError, match='max_num_split'):
            layer2(xb, a2a_ffn_overlap_degree=64)
        yb = layer2(xb, a2a_ffn_overlap_degree=32)
        assert layer2.last_stats['path'] == 'fused'
    transport.get_transport(layer2.group).check()
    assert torch.isfinite(yb.float()).all()
