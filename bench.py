#!/usr/bin/env python3
"""Headline benchmark: MoE layer forward + backward (+ SGD step) tokens/s.

Config (the reference's ``pre_test`` CLI-default shape, ``PlanMoE/examples/pre_test.py:50-60``):
per rank 16 x 512 tokens, model_dim 2048, hidden 2048, 2 local experts per GPU, top-2 gate,
capacity_factor 1.0, GELU, bf16, synthetic N(0,1) input, random-init weights, seed 0.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference|ref-torch]

``--impl reference`` builds the same layer from the reference's own package (``schemoe.moe.moe_layer``,
installed into ``baseline/_ref`` by ``baseline/build_reference.py``; nothing of this repository's package is
imported in that process), comm ``naive``, codec ``no``, its default pipeline degree 1, and runs the same step
under the same timing protocol (eager loop, one event pair per step, L2 flushed between steps).

For N > 1 launch one process per GPU with ``python -m torch.distributed.run --nproc-per-node N``.
Rank 0 prints ONE JSON line.  ``value`` is whole-job tokens/s from CUDA-event timing of exactly
K steps (max over ranks).  By default the two steps of the layer's buffer cycle (forward + backward +
SGD each) are captured once as two CUDA graphs and the K steps are K replays inside one event bracket;
a step touches about 0.6 GB, several times the L2, so no step finds its inputs cached.  The K-step bracket is repeated ``--repeats`` times and the median bracket is
reported (``spread`` holds every bracket).  ``--no-graph`` (and any run in
which capture fails) times the eager loop instead, one event pair per step with a 256 MiB L2 flush
between steps outside the brackets.  ``e2e`` repeats the measurement through the public API
including, every step, the pinned-host -> device copy of the step's input (on a copy stream, while
the step before computes) and a device -> host read of the loss.
"""

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

CFG = dict(batch=16, tokens=512, model_dim=2048, hidden=2048, local_experts=2, top_k=2,
           capacity_factor=1.0)


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=20)
    ap.add_argument('--warmup', type=int, default=5)
    ap.add_argument('--impl', default='ours', choices=['ours', 'reference', 'ref-torch'])
    ap.add_argument('--degree', default='auto', help="pipeline degree: an integer, or 'auto' for the adaptive scheduler")
    ap.add_argument('--comm', default='naive')
    ap.add_argument('--compress', default='no')
    ap.add_argument('--stages', action='store_true', help='also print per-stage device times (stderr)')
    ap.add_argument('--no-graph', action='store_true', help='time the eager loop instead of CUDA-graph replays')
    ap.add_argument('--repeats', type=int, default=5, help='how many times the K-step bracket is timed (median reported)')
    ap.add_argument('--ref-degree', type=int, default=1, help='pipeline degree of the reference arm (its default is 1)')
    return ap.parse_args()


class ClockSampler:
    """SM clock and throttle reasons of one GPU, sampled while the timed region runs.

    Reads NVML from a background thread every 5 ms (a timed region of a few tens of milliseconds
    still gets samples); falls back to ``nvidia-smi -lms 200`` when NVML cannot be loaded.  Only
    reads: no clock, power or mode setting is touched."""
    Q = ('index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,'
         'clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,'
         'clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap')

    def __init__(self, gpu_index, uuid=None):
        self.idx = gpu_index
        self.uuid = uuid
        self.proc = None
        self.path = None
        self.thread = None
        self.samples = []          # (sm_mhz, reasons bitmask)
        self.max_mhz = None
        self._stop = False

    def _nvml_loop(self, nv, h):
        while not self._stop:
            try:
                self.samples.append((nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM),
                                     nv.nvmlDeviceGetCurrentClocksEventReasons(h)))
            except Exception:
                pass
            time.sleep(0.005)

    def start(self):
        try:
            import threading
            import pynvml as nv
            nv.nvmlInit()
            h = None
            if self.uuid:
                try:
                    h = nv.nvmlDeviceGetHandleByUUID(('GPU-' + str(self.uuid)).encode())
                except Exception:
                    h = None
            if h is None:
                h = nv.nvmlDeviceGetHandleByIndex(self.idx)
            self.max_mhz = float(nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM))
            self.nv = nv
            self.thread = threading.Thread(target=self._nvml_loop, args=(nv, h), daemon=True)
            self.thread.start()
            return
        except Exception:
            self.thread = None
        try:
            fd, self.path = tempfile.mkstemp(suffix='.csv')
            os.close(fd)
            self.out = open(self.path, 'w')
            self.proc = subprocess.Popen(
                ['nvidia-smi', '-i', str(self.idx), '--query-gpu=' + self.Q, '--format=csv,noheader,nounits',
                 '-lms', '200'], stdout=self.out, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        res = {'sm_mhz': None, 'sm_max_mhz': None, 'reasons': [], 'samples': 0}
        if self.thread is not None:
            self._stop = True
            self.thread.join(timeout=2)
            nv = self.nv
            bits = {'hw_slowdown': nv.nvmlClocksEventReasonHwSlowdown,
                    'hw_thermal_slowdown': nv.nvmlClocksEventReasonHwThermalSlowdown,
                    'sw_thermal_slowdown': nv.nvmlClocksEventReasonSwThermalSlowdown,
                    'sw_power_cap': nv.nvmlClocksEventReasonSwPowerCap}
            sm = [float(c) for c, _ in self.samples]
            reasons = set()
            for _, r in self.samples:
                for n, b in bits.items():
                    if r & b:
                        reasons.add(n)
            if sm:
                res.update(sm_mhz=statistics.median(sm), sm_max_mhz=self.max_mhz, reasons=sorted(reasons),
                           samples=len(sm), source='nvml')
            return res
        if self.proc is None:
            return res
        try:
            self.proc.terminate()
            self.proc.wait(timeout=5)
        except Exception:
            pass
        try:
            self.out.close()
            rows = [r.strip().split(', ') for r in open(self.path) if r.strip()]
            os.unlink(self.path)
        except Exception:
            return res
        sm, reasons, mx = [], set(), None
        names = ['hw_slowdown', 'hw_thermal_slowdown', 'sw_thermal_slowdown', 'sw_power_cap']
        for r in rows:
            if len(r) < 9:
                continue
            try:
                sm.append(float(r[1]))
                mx = float(r[2])
            except ValueError:
                continue
            for n, v in zip(names, r[5:9]):
                if v.strip().lower().startswith('active'):
                    reasons.add(n)
        if sm:
            hi = sorted(sm)[len(sm) // 2:]          # upper half = samples under load
            res.update(sm_mhz=statistics.median(hi), sm_max_mhz=mx, reasons=sorted(reasons), samples=len(sm),
                       source='nvidia-smi')
        return res


REF_DIR = os.path.join(ROOT, 'baseline', '_ref')


def unavailable(why):
    """The reference arm's line when it cannot produce a number (one per job, also under torchrun)."""
    if int(os.environ.get('RANK', '0')) == 0:
        print(json.dumps({'impl': 'reference', 'unavailable': ' '.join(str(why).split())[:400]}))
    return 0


def pin_to_gpu_numa_node(local_rank):
    """Bind this process (and so its pinned allocations) to the CPUs next to its GPU.  Harness-level, the same
    for every arm: NVML's CPU affinity of the GPU when it can be read, otherwise an even split of the visible
    CPUs over the local ranks.  Only scheduling affinity of this process is touched."""
    try:
        import pynvml as nv
        nv.nvmlInit()
        h = nv.nvmlDeviceGetHandleByIndex(local_rank)
        words = nv.nvmlDeviceGetCpuAffinity(h, (os.cpu_count() + 63) // 64)
        cpus = {64 * w + b for w, m in enumerate(words) for b in range(64) if (m >> b) & 1}
        cpus &= os.sched_getaffinity(0)
        if cpus:
            os.sched_setaffinity(0, cpus)
            return len(cpus)
    except Exception:
        pass
    return 0


def build_ours(args, device, group_world):
    import torch
    from planmoe_b200 import moe
    degree = args.degree if args.degree in ('auto',) else int(args.degree)
    layer = moe.moe_layer(
        gate_type={'type': 'top', 'k': CFG['top_k'], 'capacity_factor': CFG['capacity_factor'], 'fp32_gate': False},
        model_dim=CFG['model_dim'],
        experts={'type': 'ffn', 'count_per_node': CFG['local_experts'], 'hidden_size_per_expert': CFG['hidden'],
                 'activation_fn': 'gelu'},
        seeds=(1, 2 + (torch.distributed.get_rank() if group_world > 1 else 0), 3),
        a2a_ffn_overlap_degree=degree, compress_name=args.compress, comm_name=args.comm)
    return layer.to(device).to(torch.bfloat16)


def build_reference(args, device, rank):
    """The reference's own layer through its own public API (``schemoe.moe.moe_layer``,
    PlanMoE/impls/moe_layer.py:44-64), imported from ``baseline/_ref`` only."""
    import torch
    import torch.nn.functional as F
    sys.path.insert(0, REF_DIR)
    for name in [m for m in sys.modules if m == 'schemoe' or m.startswith('schemoe.') or m == 'schemoe_custom_kernel']:
        del sys.modules[name]
    import schemoe
    import schemoe_custom_kernel
    for mod in (schemoe, schemoe_custom_kernel):
        where = os.path.realpath(mod.__file__)
        assert where.startswith(os.path.realpath(REF_DIR) + os.sep), 'reference imported from %s' % where
    assert not any(m == 'planmoe_b200' or m.startswith('planmoe_b200.') for m in sys.modules)
    from schemoe.moe import moe_layer
    layer = moe_layer(
        gate_type={'type': 'top', 'k': CFG['top_k'], 'capacity_factor': CFG['capacity_factor'], 'fp32_gate': False},
        model_dim=CFG['model_dim'],
        experts={'type': 'ffn', 'count_per_node': CFG['local_experts'], 'hidden_size_per_expert': CFG['hidden'],
                 'activation_fn': lambda t: F.gelu(t)},
        seeds=(1, 2 + rank, 3), a2a_ffn_overlap_degree=args.ref_degree, compress_name='no', comm_name='naive')
    return layer.to(device).to(torch.bfloat16)


class RefTorchLayer:
    """REF-TORCH: what the reference executes, restated with stock PyTorch only — ATen routing
    (one-hot masks, cumsum), index_add scatter / gather, NCCL ``all_to_all_single``, permute copies and
    ``torch.matmul`` experts, in the chunk order of ``PlanMoE/impls/overlap.py:59-74``.  Context only: the
    anchored comparison is ``--impl reference``."""

    def __init__(self, device, world):
        import torch
        torch.manual_seed(2)
        M, H, El = CFG['model_dim'], CFG['hidden'], CFG['local_experts']
        self.world = world
        self.wg = torch.nn.Parameter((torch.randn(El * world, M, device=device) * 0.02).bfloat16())
        self.w1 = torch.nn.Parameter((torch.randn(El, M, H, device=device) * 0.02).bfloat16())
        self.b1 = torch.nn.Parameter(torch.zeros(El, H, device=device).bfloat16())
        self.w2 = torch.nn.Parameter((torch.randn(El, H, M, device=device) * 0.02).bfloat16())
        self.b2 = torch.nn.Parameter(torch.zeros(El, M, device=device).bfloat16())

    def parameters(self):
        return [self.wg, self.w1, self.b1, self.w2, self.b2]

    def __call__(self, x):
        import torch
        import torch.nn.functional as F
        from planmoe_b200.ops import dispatch as D
        from planmoe_b200.impls import fast_dispatch as FD
        W = self.world
        scores = F.softmax((x @ self.wg.t()).float(), dim=1)
        from planmoe_b200.jit_kernels import gating
        gating.use_fast_cumsum = False
        crit, l_aux = FD.extract_critical(scores, CFG['top_k'], capacity_factor=CFG['capacity_factor'], alignment=4)
        plan = crit.slots
        disp = D.scatter_torch(x.float(), plan, None).to(x.dtype).view(crit[0], -1, x.size(-1))

        def a2a(t):
            if W == 1:
                return t
            from planmoe_b200.impls.communicate import all_to_all_single
            return all_to_all_single(t.contiguous())
        y = a2a(disp)
        El = y.size(0) // W
        y = y.view(W, El, -1, y.size(-1)).transpose(0, 1).contiguous().view(El, -1, y.size(-1))
        y = torch.matmul(F.gelu(torch.matmul(y, self.w1) + self.b1.unsqueeze(1)), self.w2) + self.b2.unsqueeze(1)
        y = y.view(El, W, -1, y.size(-1)).transpose(0, 1).contiguous().view(W * El, -1, y.size(-1))
        y = a2a(y)
        out = D.gather_torch(y.float().view(-1, y.size(-1)), plan, crit.stacked_gates()).to(x.dtype)
        out.l_aux = l_aux
        return out


def main():
    args = parse()
    world = int(os.environ.get('WORLD_SIZE', '1'))
    rank = int(os.environ.get('RANK', '0'))
    local_rank = int(os.environ.get('LOCAL_RANK', '0'))

    if args.impl == 'reference':
        if not os.path.isdir(os.path.join(REF_DIR, 'schemoe')):
            return unavailable('baseline/_ref is absent: the reference has not been built on this machine '
                               '(python baseline/build_reference.py --src <reference checkout>)')
        if world == 1:
            # AllToAllStatus.init returns before init_nccl when the group has one rank (PlanMoE/impls/communicate.py:
            # 218-220), the native world size stays 0 and NaiveComm::all_to_all divides the byte count by it
            # (PlanMoE/custom/comm/naive.cpp:14): an integer division by zero on the host.
            return unavailable('the reference cannot run with one rank: AllToAllStatus.init returns early for world '
                               'size 1 (communicate.py:218-220) and NaiveComm::all_to_all then divides by a world '
                               'size of 0 on the host (naive.cpp:14)')
        try:
            return run(args, world, rank, local_rank)
        except BaseException as exc:                      # build / import / run error of the reference: say which
            if isinstance(exc, (KeyboardInterrupt, SystemExit)):
                raise
            import traceback
            last = traceback.format_exception_only(type(exc), exc)[-1].strip()
            print(traceback.format_exc(), file=sys.stderr)
            return unavailable('reference failed on this box: ' + last)
    return run(args, world, rank, local_rank)


def run(args, world, rank, local_rank):
    import datetime
    import torch
    import torch.distributed as dist

    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            print('bench.py: --gpus %d needs torch.distributed.run with %d processes' % (args.gpus, args.gpus),
                  file=sys.stderr)
            return 2
    affinity_cpus = pin_to_gpu_numa_node(local_rank)
    torch.cuda.set_device(local_rank)
    device = torch.device('cuda', local_rank)
    if world > 1:
        dist.init_process_group('nccl', device_id=device, timeout=datetime.timedelta(seconds=300))

    S, M = CFG['batch'] * CFG['tokens'], CFG['model_dim']
    if args.impl == 'ours':
        layer = build_ours(args, device, world)
        params = [p for p in layer.parameters()]
        from planmoe_b200.ops import native
        launch_count = native.lib().launch_count
    elif args.impl == 'reference':
        layer = build_reference(args, device, rank)
        params = [p for p in layer.parameters()]
        launch_count = lambda: 0  # noqa: E731
    else:
        layer = RefTorchLayer(device, world)
        params = layer.parameters()
        launch_count = lambda: 0  # noqa: E731
    opt = torch.optim.SGD(params, lr=1e-4)

    torch.manual_seed(100 + rank)
    host_x = torch.randn(S, M).to(torch.bfloat16).pin_memory()
    x_dev = host_x.to(device, non_blocking=True)
    host_loss = torch.zeros(1, dtype=torch.float32).pin_memory()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    target = torch.zeros(S, M, dtype=torch.bfloat16, device=device)

    def step(x):
        opt.zero_grad(set_to_none=True)
        y = layer(x)
        loss = torch.nn.functional.mse_loss(y, target) + 0.01 * y.l_aux.to(y.dtype)
        loss.backward()
        opt.step()
        return loss

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step(x_dev)
    chosen = args.degree if args.impl == 'ours' else (args.ref_degree if args.impl == 'reference' else 1)
    sched_report = None
    if args.impl == 'ours' and args.degree == 'auto':
        # the adaptive scheduler times every candidate degree over a few steps and then freezes one;
        # keep warming up (untimed) until it has, so that the timed steps all run the frozen plan
        for _ in range(256):
            sched = getattr(layer, '_scheduler', None)
            if sched is not None and sched.frozen is not None:
                break
            step(x_dev)
        sched = getattr(layer, '_scheduler', None)
        chosen = 'auto->%s' % (sched.frozen if sched is not None else '?')
        sched_report = getattr(sched, 'report', None)
    barrier()
    if args.stages and args.impl == 'ours':
        # separate, untimed pass with per-stage CUDA events (the timed regions below run without them)
        from planmoe_b200.utils import stage_timer
        from planmoe_b200.ops import native as _native
        stage_timer.enable(True)
        for _ in range(10):
            # a delay kernel first: the host enqueues the whole step while the device waits, so the events around
            # each stage bracket kernels that run back to back (device time, not the host's launch rate)
            _native.lib().delay(4_000_000)
            step(x_dev)
        barrier()
        print('rank %d stages: %s' % (rank, json.dumps(stage_timer.summary(skip=2))), file=sys.stderr, flush=True)
        if os.environ.get('PLANMOE_GEMM_TRACE', '0') == '1':
            from planmoe_b200.ops import fused_moe
            print('rank %d trace: %s' % (rank, json.dumps(fused_moe.last_trace())), file=sys.stderr, flush=True)
        stage_timer.enable(False)
        stage_timer.reset()
    if args.impl == 'ours':
        # a bounded wait that expired during warm-up ends the run here instead of timing garbage
        from planmoe_b200.parallel import transport
        transport.get_transport(None).check()

    # ---- CUDA-graph capture of the step (two steps per graph: the layer alternates buffer sets) ------
    graphed, x_static, launches_per_step = None, None, 0
    if args.impl == 'ours' and not args.no_graph:
        try:
            from planmoe_b200.utils.graphs import GraphedSteps
            layer.l_aux = None                  # last reference to the autograd graph of the eager warm-up steps
            x_static = [x_dev.clone(), x_dev.clone()]
            turn = [0]

            def graph_step():
                loss = step(x_static[turn[0] & 1])
                turn[0] += 1
                return loss.detach().float().reshape(1)
            lc0 = launch_count()
            # one graph per step of the two-step cycle, so that the end-to-end loop can feed steps one by one
            graphed = GraphedSteps(graph_step, unroll=2, warmup=2, split=True)
            launches_per_step = (launch_count() - lc0) // (2 * 2 + 2)      # warm-up steps + the captured pair
        except Exception as exc:                                            # capture not possible: eager loop
            print('bench.py: CUDA-graph capture failed (%s); timing the eager loop' % (exc,), file=sys.stderr)
            graphed = None
            torch.cuda.synchronize()
        # every rank must take the same path from here on (the ranks' kernels wait for one another)
        agreed = torch.tensor([1 if graphed is not None else 0], device=device, dtype=torch.int32)
        if world > 1:
            dist.all_reduce(agreed, op=dist.ReduceOp.MIN)
        if int(agreed.item()) == 0:
            graphed = None
        else:
            graphed.replay()
            if args.steps & 1:
                # odd K: the last step of a bracket runs eagerly.  Warm that path after the capture (its first call
                # re-creates autograd state) and keep the layer's two-step buffer cycle intact: eager steps come in pairs.
                step(x_dev)
                step(x_dev)
        barrier()

    # ---- device-timed region: `repeats` brackets of exactly K steps each ----------------------
    sampler = ClockSampler(local_rank, getattr(torch.cuda.get_device_properties(device), 'uuid', None))
    if rank == 0:
        sampler.start()
    repeats = max(int(args.repeats), 1)
    bracket_ms, host_ms_all, launches = [], [], 0
    for _rep in range(repeats):
        l0 = launch_count()
        barrier()
        host_t0 = time.perf_counter()
        if graphed is not None:
            # K steps = K // 2 replays of the two graphs of the cycle (+ one eager step if K is odd), one event bracket
            # around all of them.  The working set of a step (about 0.6 GB of activations, receive buffers and
            # weights) is several times the 126 MB L2, so no step finds its inputs cached.
            t_s, t_e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t_s.record()
            for _ in range(args.steps // 2):
                graphed.replay()
            if args.steps & 1:
                step(x_dev)
            t_e.record()
            host_ms_all.append((time.perf_counter() - host_t0) * 1e3 / args.steps)
            if args.steps & 1:
                step(x_dev)                 # untimed: completes the buffer cycle the odd step began
            barrier()
            launches = launches_per_step * args.steps
            bracket_ms.append(t_s.elapsed_time(t_e))
            l2_note = 'working set per step (~0.6 GB) exceeds L2; K steps timed as one bracket of CUDA-graph replays'
        else:
            starts = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
            ends = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
            for i in range(args.steps):
                flush.fill_(i & 0xff)
                starts[i].record()
                step(x_dev)
                ends[i].record()
            host_ms_all.append((time.perf_counter() - host_t0) * 1e3 / args.steps)   # host time to enqueue one step
            barrier()
            launches = launch_count() - l0
            bracket_ms.append(sum(s.elapsed_time(e) for s, e in zip(starts, ends)))
            l2_note = 'flushed between timed steps (256 MiB write outside the event brackets)'
    clocks = sampler.stop() if rank == 0 else None
    host_ms = statistics.median(host_ms_all)

    # ---- end-to-end region: pinned H2D of the input + D2H of the loss, every step ---------------
    # The way a training loop feeds a GPU: the input of a later step is copied from pinned host memory on a
    # copy stream while the current step computes (a ring of device buffers), and the loss of step i is copied to
    # pinned host memory behind step i and read by the host one step later, so neither copy stalls the compute
    # stream.  Every step's input is copied and every step's loss is read inside the timed region.
    copy_stream = torch.cuda.Stream(device=device)
    cur = torch.cuda.current_stream()
    losses_read = 0
    # context for the end-to-end number (outside its timed region): what one input copy costs on this box while
    # every rank copies at once and nothing else runs
    probe = torch.empty_like(x_dev)
    barrier()
    p_s, p_e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    p_s.record()
    probe.copy_(host_x, non_blocking=True)
    p_e.record()
    p_e.synchronize()
    h2d_alone_ms = p_s.elapsed_time(p_e)
    del probe
    e2e_s = torch.cuda.Event(enable_timing=True)
    e2e_e = torch.cuda.Event(enable_timing=True)
    if graphed is not None:
        # Graph mode: step i replays graph i & 1 on static input i & 1.  The input of step i + 2 is copied host ->
        # device straight into that static input on the copy stream as soon as step i has finished with it, i.e.
        # while step i + 1 computes; the loss of a step is copied to pinned host memory behind it and read one
        # step later.
        in_ready = [torch.cuda.Event() for _ in range(2)]
        in_free = [torch.cuda.Event() for _ in range(2)]
        loss_host = [torch.zeros(1, dtype=torch.float32).pin_memory() for _ in range(2)]
        loss_done = [torch.cuda.Event() for _ in range(2)]

        def prefetch_step(i):
            p = i & 1
            with torch.cuda.stream(copy_stream):
                copy_stream.wait_event(in_free[p])       # the step that last read this input has finished
                x_static[p].copy_(host_x, non_blocking=True)
                in_ready[p].record(copy_stream)

        n_graph = args.steps - (args.steps & 1)          # the cycle has two steps: an odd last step runs eagerly
        for p in range(2):
            in_free[p].record(cur)
        barrier()
        e2e_s.record()
        for i in range(min(2, n_graph)):
            prefetch_step(i)
        for i in range(n_graph):
            p = i & 1
            cur.wait_event(in_ready[p])
            out = graphed.replay_one(p)
            in_free[p].record(cur)
            if i + 2 < n_graph:
                prefetch_step(i + 2)
            loss_host[p].copy_(out, non_blocking=True)
            loss_done[p].record(cur)
            if i > 0:
                loss_done[(i - 1) & 1].synchronize()
                _ = float(loss_host[(i - 1) & 1][0])
                losses_read += 1
        if n_graph:
            loss_done[(n_graph - 1) & 1].synchronize()
            _ = float(loss_host[(n_graph - 1) & 1][0])
            losses_read += 1
        if args.steps & 1:                             # odd K: one more step, eagerly
            cur.wait_stream(copy_stream)
            x_static[0].copy_(host_x, non_blocking=True)
            loss = step(x_static[0])
            host_loss.copy_(loss.detach().float().reshape(1), non_blocking=True)
            cur.synchronize()
            _ = float(host_loss[0])
            losses_read += 1
        e2e_e.record()
        barrier()
        assert losses_read == args.steps
        e2e_ms = e2e_s.elapsed_time(e2e_e)
    else:
        depth = 3
        x_bufs = [torch.empty_like(x_dev) for _ in range(depth)]
        x_ready = [torch.cuda.Event() for _ in range(depth)]
        x_free = [torch.cuda.Event() for _ in range(depth)]
        loss_host = [torch.zeros(1, dtype=torch.float32).pin_memory() for _ in range(2)]
        loss_done = [torch.cuda.Event() for _ in range(2)]

        def prefetch(i):
            b = i % depth
            with torch.cuda.stream(copy_stream):
                copy_stream.wait_event(x_free[b])          # the step that last read this buffer has finished
                x_bufs[b].copy_(host_x, non_blocking=True)
                x_ready[b].record(copy_stream)

        for b in range(depth):
            x_free[b].record(cur)
        barrier()
        e2e_s.record()
        for i in range(min(depth - 1, args.steps)):
            prefetch(i)
        for i in range(args.steps):
            b = i % depth
            if i + depth - 1 < args.steps:
                prefetch(i + depth - 1)
            cur.wait_event(x_ready[b])
            loss = step(x_bufs[b])
            x_free[b].record(cur)
            loss_host[i & 1].copy_(loss.detach().float().reshape(1), non_blocking=True)
            loss_done[i & 1].record(cur)
            if i > 0:                                      # read the previous step's loss while this one runs
                loss_done[(i - 1) & 1].synchronize()
                _ = float(loss_host[(i - 1) & 1][0])
                losses_read += 1
        loss_done[(args.steps - 1) & 1].synchronize()
        _ = float(loss_host[(args.steps - 1) & 1][0])
        losses_read += 1
        e2e_e.record()
        barrier()
        assert losses_read == args.steps
        e2e_ms = e2e_s.elapsed_time(e2e_e)

    if args.impl == 'ours':
        from planmoe_b200.parallel import transport
        transport.get_transport(None).check()

    t = torch.tensor(bracket_ms + [e2e_ms], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    t = t.tolist()
    bracket_ms, e2e_ms = t[:-1], t[-1]
    ms = statistics.median(bracket_ms)

    if rank == 0:
        tokens = S * world * args.steps
        out = {
            'metric': 'moe_layer_fwd_bwd_tokens_per_sec',
            'value': tokens / (ms / 1e3),
            'unit': 'tokens/s',
            'n_gpus': world, 'steps': args.steps, 'warmup': max(args.warmup, 3),
            'ms_per_step': ms / args.steps,
            'higher_is_better': True, 'scaling': 'weak', 'vs_baseline': None,
            'dtype': 'bf16', 'data': 'synthetic N(0,1) tokens, random-init weights',
            'impl': args.impl,
            'config': {
                'model': 'pre_test MoE layer: model_dim 2048, hidden 2048, 2 local experts/GPU, top-2, cf 1.0, GELU',
                'global_batch': CFG['batch'] * world, 'seq_len': CFG['tokens'],
                'parallelism': 'ep%d' % world, 'step': 'forward + backward + SGD update',
                'l2': l2_note, 'cuda_graph': graphed is not None,
                'degree': chosen, 'comm': args.comm if args.impl == 'ours' else 'naive',
                'compress': args.compress if args.impl == 'ours' else 'no',
            },
            'clocks': clocks,
            'spread': {'brackets': len(bracket_ms), 'ms_per_step': [round(b / args.steps, 5) for b in bracket_ms],
                       'min': min(bracket_ms) / args.steps, 'max': max(bracket_ms) / args.steps,
                       'reported': 'median bracket of K steps, max over ranks per bracket'},
            'e2e': {'value': tokens / (e2e_ms / 1e3), 'unit': 'tokens/s',
                    'h2d_bytes_per_step': host_x.numel() * host_x.element_size(),
                    'd2h_bytes_per_step': host_loss.numel() * host_loss.element_size(),
                    'ms_per_step': round(e2e_ms / args.steps, 5),
                    'h2d_copy_alone_ms': round(h2d_alone_ms, 4)},
            'gpu_launches': int(launches),
            'host_enqueue_ms_per_step': round(host_ms, 4),
            'cpu_affinity': affinity_cpus,
        }
        if sched_report is not None:
            out['scheduler'] = sched_report
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == '__main__':
    sys.exit(main())
