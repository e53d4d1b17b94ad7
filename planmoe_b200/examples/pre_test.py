#!/usr/bin/env python3
"""Micro-benchmark of the chunked codec + all-to-all pipeline, or of the whole MoE layer.

    torchrun --nproc_per_node=N -m planmoe_b200.examples.pre_test [flags]

Default mode measures what the reference's ``PlanMoE/examples/pre_test.py:105-224`` measures: per
step, ``degree`` chunks of a ``[E_global, capacity, model_dim]`` tensor go through
compress -> all-to-all -> decompress twice (dispatch direction and combine direction); the expert
GEMMs are optional (``--with_experts``).  The printed ``max|out - in|`` is the correctness
signal (0 for lossless codecs).  ``--layer`` instead times forward + backward of ``moe_layer``.
Flags of the reference are kept (:47-67); ``--comm`` picks the all-to-all algorithm, which the
reference hard-wires to "naive" (:198,208).  Timing is CUDA events on the device, max over ranks;
rank 0 appends one CSV row per run to ``--log``.
"""

import argparse
import math
import os
import sys

import torch
import torch.distributed as dist


def get_args(argv=None):
    p = argparse.ArgumentParser()
    p.add_argument('--local_rank', type=int, default=-1)
    p.add_argument('--batch_size', type=int, default=16)
    p.add_argument('--num_tokens', type=int, default=512)
    p.add_argument('--model_dim', type=int, default=2048)
    p.add_argument('--hidden_size', type=int, default=2048)
    p.add_argument('--num_local_experts', type=int, default=2)
    p.add_argument('--dtype', type=str, default='bfloat16')
    p.add_argument('--fp32_gate', default=False, action='store_true')
    p.add_argument('--top', type=int, default=2)
    p.add_argument('--a2a_ffn_overlap_degree', type=int, default=1)
    p.add_argument('--num_steps', type=int, default=25)
    p.add_argument('--capacity_factor', type=float, default=1.0)
    p.add_argument('--parallel_type', type=str, default='auto')
    p.add_argument('--device', type=str, default='cuda' if torch.cuda.is_available() else 'cpu')
    p.add_argument('--use_2dh', default=False, action='store_true')
    p.add_argument('--record_shapes', default=False, action='store_true')
    p.add_argument('--with_stack', default=False, action='store_true')
    p.add_argument('--log', type=str, default='test.log')
    p.add_argument('--encode', type=str, default='no')
    p.add_argument('--comm', type=str, default='naive')
    p.add_argument('--with_experts', default=False, action='store_true')
    p.add_argument('--layer', default=False, action='store_true')
    p.add_argument('--profile', default=False, action='store_true',
                   help='wrap the steps in torch.profiler and export a Chrome trace named after the config')
    return p.parse_args(argv)


def trace_handler_for(args, rank):
    def handler(prof):
        print(prof.key_averages().table(sort_by='self_cuda_time_total', row_limit=20))
        if rank == 0:
            name = 'b%d_t%d_m%d_h%d_e%d_cf%s_d%d_step%d.json' % (
                args.batch_size, args.num_tokens, args.model_dim, args.hidden_size, args.num_local_experts,
                args.capacity_factor, args.a2a_ffn_overlap_degree, prof.step_num)
            prof.export_chrome_trace(name)
    return handler


def main(argv=None):
    args = get_args(argv)
    from planmoe_b200 import moe, net, system
    from planmoe_b200.impls.overlap import ChunkHandle
    from planmoe_b200.impls import communicate as C

    backend = 'nccl' if args.device == 'cuda' else 'gloo'
    env = system.init_data_model_parallel(backend=backend) if 'RANK' in os.environ else None
    rank, world = net.get_world_rank(), net.get_world_size()
    device = torch.device('cuda', int(os.environ.get('LOCAL_RANK', 0))) if args.device == 'cuda' else torch.device('cpu')
    dtype = {'float32': torch.float32, 'float64': torch.float64, 'float16': torch.float16,
             'bfloat16': torch.bfloat16}[args.dtype]
    torch.manual_seed(0)
    say = print if rank == 0 else (lambda *a, **k: None)

    E = args.num_local_experts * world
    degree = args.a2a_ffn_overlap_degree
    align = degree * (4 if args.encode == 'zfp' else 1)
    cap = int(args.top * math.ceil(args.batch_size * args.num_tokens / E) * args.capacity_factor)
    cap = (cap + align - 1) // align * align
    say('[Benchmark] world_size = %d, dtype = %s, model_dim = %d, hidden_size = %d, samples = %d, '
        'num_local_experts = %d, topK = %d, a2a_ffn_overlap_degree = %d, capacity_factor = `%s`, device = `%s`, '
        'codec = %s, comm = %s' % (world, args.dtype, args.model_dim, args.hidden_size,
                                   args.batch_size * args.num_tokens, args.num_local_experts, args.top, degree,
                                   args.capacity_factor, device, args.encode, args.comm))

    def sync():
        if device.type == 'cuda':
            torch.cuda.synchronize()

    times = []
    if args.layer:
        layer = moe.moe_layer(
            gate_type={'type': 'top', 'k': args.top, 'capacity_factor': args.capacity_factor,
                       'fp32_gate': args.fp32_gate},
            model_dim=args.model_dim,
            experts={'type': 'ffn', 'count_per_node': args.num_local_experts,
                     'hidden_size_per_expert': args.hidden_size, 'activation_fn': 'gelu'},
            a2a_ffn_overlap_degree=degree, use_2dh=args.use_2dh, parallel_type=args.parallel_type,
            compress_name=args.encode, comm_name=args.comm, seeds=(1, rank + 1, 1)).to(device).to(dtype)
        x = torch.randn(args.batch_size * args.num_tokens, args.model_dim, device=device, dtype=dtype,
                        requires_grad=True)

        def step():
            y = layer(x)
            (y.float().sum() + y.l_aux.float()).backward()
            return None
    else:
        x = torch.randn(E, cap, args.model_dim, device=device, dtype=dtype)
        w1 = torch.randn(args.num_local_experts, args.model_dim, args.hidden_size, device=device, dtype=dtype) * 0.02
        w2 = torch.randn(args.num_local_experts, args.hidden_size, args.model_dim, device=device, dtype=dtype) * 0.02
        C.AllToAllStatus.init(None, degree, 1)

        def step():
            chunks = [c.contiguous() for c in x.split(cap // degree, dim=1)]
            pend = [ChunkHandle(args.encode, args.comm, None).launch(c) for c in chunks]
            for i in range(degree):
                t = pend[i].finish()
                if args.with_experts:
                    t = C.pre_expert_permute(t)
                    t = torch.relu(torch.matmul(t, w1))
                    t = torch.matmul(t, w2)
                    t = C.post_expert_permute(t)
                pend[i] = ChunkHandle(args.encode, args.comm, None).launch(t.contiguous())
            out = torch.cat([p.finish() for p in pend], dim=1)
            return out

    prof = None
    if args.profile:
        from torch.profiler import ProfilerActivity, profile, schedule
        prof = profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA],
                       schedule=schedule(wait=1, warmup=2, active=3), record_shapes=args.record_shapes,
                       with_stack=args.with_stack, on_trace_ready=trace_handler_for(args, rank))
        prof.start()

    err = None
    for it in range(args.num_steps):
        sync()
        if device.type == 'cuda':
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            out = step()
            e.record()
            sync()
            ms = s.elapsed_time(e)
        else:
            t0 = system.record_time(is_cuda=False)
            out = step()
            ms = (system.record_time(is_cuda=False) - t0) * 1e3
        t = torch.tensor([ms], device=device, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        times.append(float(t))
        if out is not None and not args.with_experts and it == 0:
            err = float((out.float() - x.float()).abs().max())
            say('max|out - in| = %g' % err)
        if prof is not None:
            prof.step()
        net.barrier()
    if prof is not None:
        prof.stop()

    kept = times[5:] if len(times) > 5 else times
    mean = sum(kept) / len(kept)
    payload = x.numel() * x.element_size()
    say('mean step %.3f ms over %d steps (first 5 dropped); payload %.1f MiB/rank/direction' % (
        mean, len(kept), payload / 2 ** 20))
    if not args.layer and world > 1:
        say('a2a algbw %.1f GB/s, busbw %.1f GB/s (2 exchanges per step, codec included)' % (
            2 * payload / mean / 1e6, 2 * payload / mean / 1e6 * (world - 1) / world))
    if rank == 0:
        with open(args.log, 'a+') as f:
            f.write('%d,%d,%d,%d,%s,%s,%s,%d,%s\n' % (args.batch_size, args.num_tokens, args.model_dim,
                                                     args.hidden_size, args.comm, args.encode, args.capacity_factor,
                                                     degree, kept))
    if device.type == 'cuda' and world > 1:
        from planmoe_b200.parallel import transport
        transport.get_transport(None).check()
    return mean, err


if __name__ == '__main__':
    main()
    if dist.is_available() and dist.is_initialized():
        dist.destroy_process_group()
