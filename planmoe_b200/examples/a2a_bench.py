#!/usr/bin/env python3
"""All-to-all sweep: bus bandwidth of every algorithm of the symmetric-heap transport against NCCL.

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 \
        -m planmoe_b200.examples.a2a_bench [--sizes-mb 1,4,16,64,256] [--algos flat,pipe,dd,hetu,nccl]
        [--codecs no,int8] [--iters 10] [--groups 2]

Per rank a bf16 ~N(0,1) tensor of ``size`` bytes, viewed as rows of 1024 elements, is exchanged so
that every rank receives an equal slice from every other rank.  ``flat`` / ``pipe`` / ``dd`` /
``hetu`` are the in-kernel peer-store algorithms (``parallel/a2a.py``); ``pipe``, ``dd`` and ``hetu``
run on ``--groups`` logical groups of N / groups ranks each (``LOCAL_SIZE``), the way the reference's
Pipe-A2A, 2DH and HeTu algorithms see nodes.  ``nccl`` is ``dist.all_to_all_single``, the transport
the reference builds from grouped ncclSend / ncclRecv (``PlanMoE/custom/comm/naive.cpp:11-27``).
With ``int8`` the timed region is encode -> exchange of the packed tensors -> decode, and the
bandwidth is quoted on the raw bf16 bytes.

Timing: CUDA events around each exchange on every rank after 3 warm-up exchanges, a 256 MiB write
between iterations to flush L2, mean over ``--iters``, MAX over ranks.  bus GB/s =
bytes * (N - 1) / N / time; rank 0 prints one JSON line per case.
"""

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

NVLINK_NOMINAL_GBS = 900.0       # per direction per GPU
NVLINK_MEASURED_GBS = 770.0      # peer copy measured on this pool, per direction


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument('--sizes-mb', default='1,4,16,64,256')
    ap.add_argument('--algos', default='flat,pipe,dd,hetu,nccl')
    ap.add_argument('--codecs', default='no,int8')
    ap.add_argument('--iters', type=int, default=10)
    ap.add_argument('--groups', type=int, default=2)
    args = ap.parse_args(argv)

    rank, world = int(os.environ.get('RANK', 0)), int(os.environ.get('WORLD_SIZE', 1))
    local_rank = int(os.environ.get('LOCAL_RANK', 0))
    torch.cuda.set_device(local_rank)
    dev = torch.device('cuda', local_rank)
    if world > 1:
        dist.init_process_group('nccl', device_id=dev)
    if world % max(args.groups, 1) == 0 and world > args.groups:
        os.environ['LOCAL_SIZE'] = str(world // args.groups)

    from planmoe_b200.parallel import codecs, transport
    tr = transport.get_transport(None)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def exchange(t, algo):
        if algo == 'nccl':
            if world == 1:
                return t.clone()
            out = torch.empty_like(t)
            dist.all_to_all_single(out, t)
            return out
        return tr.all_to_all(t, algo)

    def run_case(size_mb, algo, codec_name):
        nbytes = size_mb << 20
        rows = nbytes // 2 // 1024
        rows -= rows % world
        torch.manual_seed(7 + rank)
        x = torch.randn(rows, 1024, device=dev).to(torch.bfloat16)
        comp = codecs.get_compressor(codec_name)

        def once():
            if codec_name == 'no':
                return exchange(x, algo), x.numel() * 2
            packed = comp.compress(x, world)
            wires = [exchange(w.view(world, -1), algo).view(w.shape) for w in packed.wires]
            wire_bytes = packed.wire_bytes()
            return comp.decompress(codecs.Packed(wires, packed.meta)), wire_bytes

        for _ in range(3):
            out, wire_bytes = once()
        # correctness: what arrived from rank s is the slice that rank s addressed to me
        ok = True
        if codec_name == 'no' and world > 1:
            ref = torch.empty_like(x)
            dist.all_to_all_single(ref, x)
            ok = bool(torch.equal(out, ref))
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        total = 0.0
        for i in range(args.iters):
            flush.fill_(i & 0xff)
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            once()
            e.record()
            e.synchronize()
            total += s.elapsed_time(e)
        t = torch.tensor([total / args.iters], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        tr.check()
        ms = float(t.item())
        raw = x.numel() * 2
        bus = raw * (world - 1) / max(world, 1) / (ms * 1e-3) / 1e9
        if rank == 0:
            print(json.dumps({
                'case': 'a2a', 'gpus': world, 'groups': args.groups if 'LOCAL_SIZE' in os.environ else 1,
                'algo': algo, 'codec': codec_name, 'payload_mb': size_mb, 'wire_bytes': int(wire_bytes),
                'ms': round(ms, 4), 'bus_gbs': round(bus, 1),
                'of_900_nominal': round(bus / NVLINK_NOMINAL_GBS, 3),
                'of_770_measured': round(bus / NVLINK_MEASURED_GBS, 3), 'matches_nccl': ok}), flush=True)

    for size_mb in [int(s) for s in args.sizes_mb.split(',') if s]:
        for codec_name in args.codecs.split(','):
            for algo in args.algos.split(','):
                run_case(size_mb, algo, codec_name)
    if world > 1:
        dist.destroy_process_group()


if __name__ == '__main__':
    main()
