#!/usr/bin/env python3
"""All-to-all sweep: bus bandwidth of every algorithm of the symmetric-heap transport against NCCL.

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 \
        -m planmoe_b200.examples.a2a_bench [--sizes-mb 1,4,16,64,256,1024] [--algos flat,pipe,dd,hetu,nccl]
        [--codecs no,int8] [--iters 20] [--groups 2] [--heap-out]

Per rank a bf16 ~N(0,1) tensor of ``size`` bytes, viewed as rows of 1024 elements, is exchanged so
that every rank receives an equal slice from every other rank.  ``flat`` / ``pipe`` / ``dd`` /
``hetu`` are the in-kernel peer-store algorithms (``parallel/a2a.py``); ``pipe``, ``dd`` and ``hetu``
run on ``--groups`` logical groups of N / groups ranks each (``LOCAL_SIZE``), the way the reference's
Pipe-A2A, 2DH and HeTu algorithms see nodes.  ``nccl`` is ``dist.all_to_all_single``, the transport
the reference builds from grouped ncclSend / ncclRecv (``PlanMoE/custom/comm/naive.cpp:11-27``).
With ``int8`` the timed region is encode -> exchange of the packed tensors -> decode, and the
bandwidth is quoted on the raw bf16 bytes.  ``--heap-out`` returns the result as a view of the receive
buffer in the symmetric heap instead of copying it out (see ``parallel/a2a.py`` for its lifetime).

Protocol: every (size, codec, algorithm) cell is warmed up on its own (3 exchanges) and then timed for
``--iters`` exchanges, each between CUDA events, with a 256 MiB write in between to flush L2; per iteration the
MAX over ranks is taken, and the median and minimum over iterations are reported.  The order of the algorithms
inside a (size, codec) group is shuffled (same seed on every rank) so that no algorithm always runs first.  Cells
that execute the same message plan on the same kernel (``flat``, ``pipe`` and ``dd`` when there is one group, or
one rank per group) must agree within 5 % of each other: a larger spread is reported as ``plan_mismatch``.
bus GB/s = bytes * (N - 1) / N / time; rank 0 prints one JSON line per cell.
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
    import random
    import statistics
    ap = argparse.ArgumentParser()
    ap.add_argument('--sizes-mb', default='1,4,16,64,256')
    ap.add_argument('--algos', default='flat,pipe,dd,hetu,nccl')
    ap.add_argument('--codecs', default='no,int8')
    ap.add_argument('--iters', type=int, default=20)
    ap.add_argument('--groups', type=int, default=2)
    ap.add_argument('--heap-out', action='store_true')
    ap.add_argument('--seed', type=int, default=0)
    args = ap.parse_args(argv)

    rank, world = int(os.environ.get('RANK', 0)), int(os.environ.get('WORLD_SIZE', 1))
    local_rank = int(os.environ.get('LOCAL_RANK', 0))
    torch.cuda.set_device(local_rank)
    dev = torch.device('cuda', local_rank)
    if world > 1:
        dist.init_process_group('nccl', device_id=dev)
    grouped = world % max(args.groups, 1) == 0 and world > args.groups
    if grouped:
        os.environ['LOCAL_SIZE'] = str(world // args.groups)
    local = world // args.groups if grouped else world

    from planmoe_b200.parallel import codecs, transport
    tr = transport.get_transport(None)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def exchange(t, algo, var_len=None):
        if algo == 'nccl':
            if world == 1:
                return t.clone()
            out = torch.empty_like(t)
            dist.all_to_all_single(out, t)
            return out
        return tr.all_to_all(t, algo, var_len=var_len, heap_out=args.heap_out and var_len is None)

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
            return comp.decompress(codecs.Packed(wires, packed.meta)), sum(w.numel() * w.element_size() for w in wires)

        for _ in range(3):
            out, wire_bytes = once()
        # correctness: what arrived from rank s is the slice that rank s addressed to me
        ok = True
        if codec_name == 'no' and world > 1:
            ref = torch.empty_like(x)
            dist.all_to_all_single(ref, x)
            ok = bool(torch.equal(out, ref))
        del out
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        times = []
        for i in range(args.iters):
            flush.fill_(i & 0xff)
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            once()
            e.record()
            e.synchronize()
            times.append(s.elapsed_time(e))
        t = torch.tensor(times, device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        tr.check()
        times = t.tolist()
        med, best = statistics.median(times), min(times)
        raw = x.numel() * 2

        def bus(ms):
            return raw * (world - 1) / max(world, 1) / (ms * 1e-3) / 1e9
        rec = {'case': 'a2a', 'gpus': world, 'groups': args.groups if grouped else 1,
               'algo': algo, 'codec': codec_name, 'payload_mb': size_mb, 'wire_bytes': int(wire_bytes),
               'ms_median': round(med, 4), 'ms_min': round(best, 4), 'bus_gbs': round(bus(med), 1),
               'bus_gbs_best': round(bus(best), 1), 'of_900_nominal': round(bus(med) / NVLINK_NOMINAL_GBS, 3),
               'of_770_measured': round(bus(med) / NVLINK_MEASURED_GBS, 3), 'matches_nccl': ok,
               'heap_out': bool(args.heap_out and algo != 'nccl' and codec_name == 'no')}
        return rec

    same_plan = {'flat', 'pipe', 'dd'} if (local == world or local == 1) else set()
    rng = random.Random(args.seed)
    for size_mb in [int(s) for s in args.sizes_mb.split(',') if s]:
        for codec_name in args.codecs.split(','):
            algos = [a for a in args.algos.split(',') if a]
            rng.shuffle(algos)
            recs = [run_case(size_mb, algo, codec_name) for algo in algos]
            shared = [r['ms_median'] for r in recs if r['algo'] in same_plan]
            mismatch = len(shared) > 1 and max(shared) > 1.05 * min(shared)
            for r in sorted(recs, key=lambda r: r['algo']):
                if r['algo'] in same_plan and len(shared) > 1:
                    r['plan_mismatch'] = bool(mismatch)
                if rank == 0:
                    print(json.dumps(r), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == '__main__':
    main()
