"""Rank-side bodies of the multi-process tests (see mp_util.run_workers)."""

import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, HERE)

import torch
import torch.distributed as dist
import torch.nn.functional as F


def _init():
    if os.environ.get('PLANMOE_USER_COMM_SO'):           # an out-of-tree C++ comm to register before use
        import ctypes
        from planmoe_b200.ops import native
        native.lib()
        ctypes.CDLL(os.environ['PLANMOE_USER_COMM_SO'], mode=ctypes.RTLD_GLOBAL)
    backend = os.environ.get('MP_BACKEND', 'gloo')
    rank, world = int(os.environ['RANK']), int(os.environ['WORLD_SIZE'])
    if backend == 'nccl':
        torch.cuda.set_device(int(os.environ['LOCAL_RANK']))
        dist.init_process_group('nccl', device_id=torch.device('cuda', int(os.environ['LOCAL_RANK'])))
        dev = torch.device('cuda', int(os.environ['LOCAL_RANK']))
    else:
        dist.init_process_group('gloo')
        dev = torch.device('cpu')
    return rank, world, dev


def _gather_cat(t):
    out = [torch.empty_like(t) for _ in range(dist.get_world_size())]
    dist.all_gather(out, t.contiguous())
    return torch.cat(out, dim=0)


def _layer_vs_oracle(dev, dtype, comm, compress, degree, tol, gtol=None, E_l=2, M=64, H=96, S=96, act='relu', k=2, cf=2.0):
    """Expert-parallel layer on W ranks against the dense per-token oracle evaluated with all
    experts' weights gathered; expert grads are compared after summing the oracle's over ranks."""
    from planmoe_b200 import moe
    from oracle import dense_moe_reference
    rank, world = dist.get_rank(), dist.get_world_size()
    layer = moe.moe_layer(
        gate_type={'type': 'top', 'k': k, 'capacity_factor': cf, 'fp32_gate': True}, model_dim=M,
        experts={'type': 'ffn', 'count_per_node': E_l, 'hidden_size_per_expert': H, 'activation_fn': act},
        seeds=(1, 10 + rank, 3), a2a_ffn_overlap_degree=degree, comm_name=comm, compress_name=compress)
    layer = layer.to(dev).to(dtype)
    layer.gates[0].wg.float()
    torch.manual_seed(100 + rank)
    x = torch.randn(S, M, device=dev).to(dtype).requires_grad_(True)
    y = layer(x)
    w = torch.linspace(-1, 1, y.numel(), device=dev).view_as(y)
    ((y.float() * w).sum() + y.l_aux.float()).backward()
    if dev.type == 'cuda':
        from planmoe_b200.parallel import transport
        transport.get_transport(layer.group).check()

    ex = layer.experts
    full = [_gather_cat(p.detach().float()).cpu().requires_grad_(True)
            for p in (ex.batched_fc1_w, ex.batched_fc1_bias, ex.batched_fc2_w, ex.batched_fc2_bias)]
    wg = layer.gates[0].wg.weight.detach().float().cpu().requires_grad_(True)
    xr = x.detach().float().cpu().requires_grad_(True)
    fn = {'relu': F.relu, 'gelu': F.gelu}[act]
    yr, l_aux = dense_moe_reference(xr, wg, *full, top_k=k, capacity_factor=cf, act=fn, alignment=4 * degree)
    ((yr * w.cpu().float()).sum() + l_aux).backward()

    def close(a, b, what):
        a, b = a.detach().float().cpu(), b.detach().float()
        err = ((a - b).abs().max() / (b.abs().max() + 1e-6)).item()
        limit = tol if what == 'y' or gtol is None else gtol
        assert err < limit, (what, err)

    close(y, yr, 'y')
    close(x.grad, xr.grad, 'dx')
    close(layer.gates[0].wg.weight.grad, wg.grad, 'dwg')
    for p, f, name in zip((ex.batched_fc1_w, ex.batched_fc1_bias, ex.batched_fc2_w, ex.batched_fc2_bias), full,
                          ('dw1', 'db1', 'dw2', 'db2')):
        g = f.grad.clone().to(dev if dev.type == 'cuda' else 'cpu')
        dist.all_reduce(g)
        close(p.grad, g[rank * E_l:(rank + 1) * E_l].cpu(), name)


def cpu_layer(comm='naive', compress='no', degree='1'):
    rank, world, dev = _init()
    lossless = compress in ('no', 'lz')
    tol = 1e-4 if lossless else 0.15
    # a lossy codec also quantises the gradients that travel back: looser bound on grads
    _layer_vs_oracle(dev, torch.float32, comm, compress, int(degree), tol, gtol=None if lossless else 0.4)


def cpu_collectives():
    rank, world, dev = _init()
    from planmoe_b200 import net
    x = torch.arange(world * 6, dtype=torch.float32).view(world * 2, 3) + 100 * rank
    x.requires_grad_(True)
    y = net.all_to_all(x, 1, 0)             # gather dim 1, scatter dim 0
    assert y.shape == (2, 3 * world)
    y.sum().backward()
    assert torch.equal(x.grad, torch.ones_like(x))
    z = net.all_to_all(net.all_to_all(x.detach(), 1, 0), 0, 1)
    assert torch.equal(z, x.detach())
    g = net.simple_all_gather(torch.full((2,), float(rank)))
    assert g.tolist() == [float(r) for r in range(world) for _ in range(2)]
    rs = net.simple_reduce_scatter(torch.ones(world * 2))
    assert rs.tolist() == [float(world)] * 2
    assert torch.equal(net.simple_split(torch.arange(world * 2)), torch.arange(world * 2)[rank * 2:rank * 2 + 2])
    v = torch.ones(3, requires_grad=True)
    net.allreduce_backward(v).sum().backward()
    assert v.grad.tolist() == [float(world)] * 3
    assert net.allreduce_forward(torch.ones(1)).item() == world
    # ZeRO helper: shard, gather back
    p = torch.arange(7, dtype=torch.float32)
    shard, shape = net.zero_scatter(p, net.simple_split)
    back = net.zero_gather(shard, full_shape=list(shape))
    assert torch.equal(back, p)
    groups = net.create_groups_from_world(group_count=2) if world % 2 == 0 else None
    if groups is not None:
        assert groups.model_size == world // 2 and groups.group_count == 2
    net.barrier()


def cpu_async_a2a_functions():
    """Chunked scatter / gather all-to-all Functions and the stream hand-over Functions against plain
    all_to_all_single, forward and backward."""
    from planmoe_b200.impls import communicate as C
    rank, world, dev = _init()
    C.AllToAllStatus.init(None, 2, 1)
    torch.manual_seed(rank)
    x = torch.randn(world * 2, 4, 3, device=dev, requires_grad=True)
    ref = torch.empty_like(x)
    dist.all_to_all_single(ref, x.detach().contiguous())
    chunks = C.AllToAllScatterAsync.apply(C.CurrentStreamRelease.apply(x, 0), False)
    assert len(chunks) == 2 and chunks[0].shape == (world * 2, 2, 3)
    assert torch.equal(torch.cat(chunks, dim=1), ref)
    back = C.CurrentStreamAcquire.apply(C.AllToAllGatherAsync.apply(False, *chunks), 1)
    assert torch.allclose(back, x.detach())                 # a2a of an a2a with equal splits is the identity
    w = torch.arange(back.numel(), dtype=back.dtype).view_as(back)
    (back * w).sum().backward()
    assert torch.allclose(x.grad, w)
    y = C.AllToAll2DAsync.apply(x.detach())
    assert torch.equal(y, ref)
    print('async a2a functions ok')


def cpu_checkpoint_gather_and_reload():
    """Per-rank shards -> full state (all_gather) -> shards of a world of another size -> same tensors."""
    import tempfile
    from planmoe_b200 import moe
    from planmoe_b200.utils import checkpoint as ck
    rank, world, dev = _init()
    layer = moe.moe_layer(gate_type={'type': 'top', 'k': 2}, model_dim=16,
                          experts={'type': 'ffn', 'count_per_node': 2, 'hidden_size_per_expert': 24,
                                   'activation_fn': 'relu'}, seeds=(1, 10 + rank, 3))
    full = ck.gather_expert_state(layer.state_dict())
    assert full['experts.batched_fc1_w'].shape[0] == 2 * world
    mine = ck.shard_expert_state(full, rank, world)
    for k, v in layer.state_dict().items():
        assert torch.equal(mine[k], v), k
    # a world of half the size would hold twice the experts per rank, in global expert order
    half = ck.shard_expert_state(full, 0, max(world // 2, 1))
    assert torch.equal(half['experts.batched_fc1_w'][:2], full['experts.batched_fc1_w'][:2])
    prefix = os.path.join(tempfile.gettempdir(), 'planmoe_ck_%s' % os.environ['MASTER_PORT'])
    ck.save_sharded(layer, prefix)
    dist.barrier()
    other = moe.moe_layer(gate_type={'type': 'top', 'k': 2}, model_dim=16,
                          experts={'type': 'ffn', 'count_per_node': 2, 'hidden_size_per_expert': 24,
                                   'activation_fn': 'relu'}, seeds=(5, 50 + rank, 7))
    ck.load_sharded(other, prefix)
    for (k, a), (_, b) in zip(layer.state_dict().items(), other.state_dict().items()):
        assert torch.equal(a, b), k
    dist.barrier()
    os.remove('%s.rank%d-of-%d.pt' % (prefix, rank, world))
    print('checkpoint helpers ok')


def cpu_zero_optimizer():
    rank, world, dev = _init()
    from planmoe_b200 import net
    torch.manual_seed(0)
    w = torch.nn.Parameter(torch.randn(5, 3))
    e = torch.nn.Parameter(torch.randn(2, 2))
    e._tutel_expert = True
    ref_w = w.detach().clone()
    opt = net.TutelDistributedOptimizer([w, e], average_shared=True).warp_local(torch.optim.SGD, lr=0.5)
    loss = (w * (rank + 1)).sum() + e.sum()
    loss.backward()
    opt.step()
    mean_grad = sum(r + 1 for r in range(world)) / world
    assert torch.allclose(w.data, ref_w - 0.5 * mean_grad, atol=1e-6)
    opt.zero_grad()
    assert float(w.grad.abs().sum()) == 0.0


def cpu_sharded_experts(mode='model'):
    """Fewer experts than ranks: both sharding modes give what one unsharded expert set gives."""
    rank, world, dev = _init()
    from planmoe_b200 import moe
    torch.manual_seed(0)
    M, H = 16, 8 * world
    layer = moe.moe_layer({'type': 'top', 'k': 1, 'capacity_factor': 4.0}, M,
                          experts={'type': 'ffn', 'count_per_node': -world, 'hidden_size_per_expert': H,
                                   'activation_fn': 'relu'},
                          seeds=(1, 2, 3), parallel_type=mode)
    assert layer.num_global_experts == 1 and layer.sharded_count == world
    # make shards slices of one common expert
    torch.manual_seed(7)
    W1, B1, W2, B2 = torch.randn(1, M, H), torch.randn(1, H), torch.randn(1, H, M), torch.randn(1, M)
    hs = H // world
    ex = layer.experts
    with torch.no_grad():
        ex.batched_fc1_w.copy_(W1[:, :, rank * hs:(rank + 1) * hs])
        ex.batched_fc1_bias.copy_(B1[:, rank * hs:(rank + 1) * hs])
        ex.batched_fc2_w.copy_(W2[:, rank * hs:(rank + 1) * hs])
        width = ex.batched_fc2_bias.size(1)
        ex.batched_fc2_bias.copy_(B2[:, rank * width:(rank + 1) * width])
    torch.manual_seed(50 + rank)
    x = torch.randn(12, M)
    y = layer(x)
    ref = (F.relu(x @ W1[0] + B1[0]) @ W2[0] + B2[0])        # softmax over one expert: gate == 1
    assert torch.allclose(y, ref, atol=1e-4, rtol=1e-4), (y - ref).abs().max()


def cpu_rank_never_joins():
    """Failure on the host: the last rank exits before the collective; the others get an error from
    the process group's timeout instead of hanging."""
    import datetime
    rank, world = int(os.environ['RANK']), int(os.environ['WORLD_SIZE'])
    dist.init_process_group('gloo', timeout=datetime.timedelta(seconds=5))
    if rank == world - 1:
        os._exit(0)
    try:
        t = torch.ones(world * 4)
        out = torch.empty_like(t)
        dist.all_to_all_single(out, t)
    except Exception as ex:          # expected: timeout / connection closed
        print('caught', type(ex).__name__)
        os._exit(0)
    raise SystemExit('collective with a missing rank did not fail')


def gpu_layer(comm='naive', compress='no', degree='1', fused='1'):
    rank, world, dev = _init()
    os.environ['PLANMOE_FUSED'] = fused
    _layer_vs_oracle(dev, torch.bfloat16, comm, compress, int(degree), 6e-2,
                     gtol=None if compress in ('no', 'lz') else 0.4, E_l=2, M=256, H=256, S=1024, act='gelu', cf=1.0)
    dist.barrier()


def gpu_a2a(algo='flat'):
    rank, world, dev = _init()
    from planmoe_b200.parallel import transport
    tr = transport.get_transport(None)
    for it, nelem in enumerate([4096, 1 << 20, 4096, 3 << 19]):
        torch.manual_seed(rank * 100 + it)
        x = torch.randn(world, nelem, device=dev).to(torch.bfloat16)
        ref = torch.empty_like(x)
        dist.all_to_all_single(ref, x)
        out = tr.all_to_all(x, algo)
        tr.check()
        assert torch.equal(out, ref), (algo, it, rank)
    dist.barrier()


def gpu_native_comm_a2a(comm='native_flat'):
    """A C++ comm object against all_to_all_single: several sizes, buffers reused, sizes growing."""
    rank, world, dev = _init()
    from planmoe_b200.parallel import comms, transport
    for it, nelem in enumerate([4096, 1 << 18, 4096, 3 << 18, 1 << 18]):
        torch.manual_seed(rank * 100 + it)
        x = torch.randn(world, nelem, device=dev).to(torch.bfloat16)
        ref = torch.empty_like(x)
        dist.all_to_all_single(ref, x)
        c = comms.get_comm(comm)
        assert isinstance(c, comms.NativeComm)
        out = c.all_to_all(x)
        transport.get_transport(None).check()
        assert torch.equal(out, ref), (comm, it, rank)
    dist.barrier()


def gpu_codec_comm_pipeline(comm='pipe', compress='int8'):
    rank, world, dev = _init()
    from planmoe_b200.impls.overlap import ChunkHandle
    torch.manual_seed(7 + rank)                        # every rank's data (and compressed size) differs
    for it, rows in enumerate((64, 8, 64)):            # buffers of the channel are reused across sizes
        x = F.relu(torch.randn(world * 2, rows, 256, device=dev) - 0.3 * rank).to(torch.bfloat16)
        h = ChunkHandle(compress, comm, None).launch(x)
        y = h.finish()
        ref = torch.empty_like(x)
        dist.all_to_all_single(ref, x)
        torch.cuda.synchronize()
        from planmoe_b200.parallel import transport
        transport.get_transport(None).check()
        err = (y.float() - ref.float()).abs().max().item()
        _check_codec_err(err, ref, compress)
    dist.barrier()


def _check_codec_err(err, ref, compress):
    lossless = compress in ('no', 'lz')
    assert err <= (0.0 if lossless else (0.1 if compress == 'zfp' else 0.02) * ref.float().abs().max().item()), err


if __name__ == '__main__':
    fn = sys.argv[1]
    globals()[fn](*sys.argv[2:])
    if dist.is_initialized():
        dist.destroy_process_group()
