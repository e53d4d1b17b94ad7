#!/usr/bin/env python3
"""Per-kernel timing on one GPU with CUDA events, reported against the measured peaks.

    python -m planmoe_b200.examples.kernel_bench [--case NAME] [--iters N] [--small]

Cases: gemm_fwd (K-major x MN-major, bias+GELU epilogue), gemm_push (same GEMM, rows stored into the
symmetric heap with flags), gemm_dgrad (K x K, activation-backward
epilogue), gemm_wgrad (MN x MN), cublas (torch.bmm of the forward shape, for comparison), scatter
(dispatch), gather (combine), gate (fused gate), int8 (encode + decode), misc (the small kernels: wire-row int8
encoder, batch-prioritised order, slot-map build / remap, cumsum, flag wait, delay, allocation-free column sum), all.  Shapes are the
per-rank shapes of the pre_test layer: 2 experts x 8192 rows, model_dim = hidden = 2048
(``--small`` quarters the rows so that a profiler capture stays short).  Between timed
iterations a 256 MiB buffer is written to flush L2.  One JSON line per case.
"""

import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from planmoe_b200.ops import gemm, native  # noqa: E402


def peaks():
    path = os.path.join(ROOT, 'MEASURED_PEAKS.json')
    if os.path.exists(path):
        p = json.load(open(path))
        return p['hbm_gbs'], p['bf16_tflops'], 'measured'
    return 6650.0, 1590.0, 'fallback'


def timed(fn, iters, flush):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    best = 1e9
    for i in range(iters):
        flush.fill_(i & 0xff)
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        ms = s.elapsed_time(e)
        total += ms
        best = min(best, ms)
    return total / iters, best


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--case', default='all')
    ap.add_argument('--iters', type=int, default=10)
    ap.add_argument('--small', action='store_true')
    ap.add_argument('--act', type=int, default=2, help='activation of the gemm_fwd / gemm_dgrad epilogues: 0 identity, 1 ReLU, 2 GELU, 3 SiLU')
    ap.add_argument('--no-aux', action='store_true', help='gemm_fwd without the saved-derivative output')
    ap.add_argument('--trace', action='store_true',
                    help='GEMM cases: one extra launch with the role trace; prints where the first epilogue warp waited')
    args = ap.parse_args()
    lib = native.lib()
    hbm, tf, how = peaks()
    dev = 'cuda'
    G, R, M, H = 2, (2048 if args.small else 8192), 2048, 2048
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    bf = torch.bfloat16
    x = torch.randn(G, R, M, device=dev).to(bf)
    w1 = (torch.randn(G, M, H, device=dev) * 0.02).to(bf)
    b1 = torch.zeros(G, H, device=dev, dtype=bf)
    dy = torch.randn(G, R, H, device=dev).to(bf)
    pre = torch.empty(G, R, H, device=dev, dtype=bf)
    out = torch.empty(G, R, H, device=dev, dtype=bf)
    flops = 2.0 * G * R * M * H

    def report(name, ms, best, flop=None, bytes_=None):
        rec = {'case': name, 'ms_mean': round(ms, 4), 'ms_best': round(best, 4), 'rows': R}
        if flop:
            rec['tflops'] = round(flop / best / 1e9, 1)
            rec['frac_of_%s_bf16_peak' % how] = round(flop / best / 1e9 / tf, 3)
        if bytes_:
            rec['gbs'] = round(bytes_ / best / 1e6, 1)
            rec['frac_of_%s_hbm' % how] = round(bytes_ / best / 1e6 / hbm, 3)
        print(json.dumps(rec), flush=True)

    cases = args.case.split(',')
    want = lambda c: 'all' in cases or c in cases  # noqa: E731

    def traced(name, fn):
        """fn(trace_ptr=...) launches one GEMM; report the epilogue's waits as fractions of its tile loop."""
        if not args.trace:
            return
        tb = torch.zeros(296, 32, dtype=torch.int64, device=dev)
        fn(trace_ptr=tb.data_ptr())
        torch.cuda.synchronize()
        t = tb[tb[:, 4] > 0]
        loop = (t[:, 7] >> 32).float()
        stage = (t[:, 7] & 0xffffffff).float()
        acc = t[:, 6].float()
        print(json.dumps({'case': name + '_trace', 'ctas': int(t.size(0)),
                          'kernel_us_max': round(float((t[:, 4] - t[:, 0]).max()) / 1e3, 1),
                          'epi_loop_mclk_mean': round(float(loop.mean()) / 1e6, 4),
                          'wait_acc_frac': round(float((acc / loop).mean()), 3),
                          'wait_staging_frac': round(float((stage / loop).mean()), 3)}), flush=True)

    if want('gemm_fwd'):
        ms, best = timed(lambda: gemm.grouped_gemm(x, False, w1, True, gemm.EPI_BIAS_ACT, args.act, bias=b1, aux=None if args.no_aux else pre, out=out),
                         args.iters, flush)
        report('gemm_fwd' if args.act == 2 else 'gemm_fwd_act%d' % args.act, ms, best, flops)
        traced('gemm_fwd', lambda **kw: gemm.grouped_gemm(x, False, w1, True, gemm.EPI_BIAS_ACT, args.act, bias=b1, aux=None if args.no_aux else pre,
                                                          out=out, **kw))
    if want('gemm_plain'):
        ms, best = timed(lambda: gemm.grouped_gemm(x, False, w1, True, out=out), args.iters, flush)
        report('gemm_plain', ms, best, flops)
        traced('gemm_plain', lambda **kw: gemm.grouped_gemm(x, False, w1, True, out=out, **kw))
    if want('gemm_push'):
        # push epilogue with this rank's own heap as the destination (one rank: no NVLink traffic)
        from planmoe_b200.parallel import transport
        tr = transport.get_transport(None)
        blk = tr.alloc(G * R * H * 2 + 4096)
        ms, best = timed(lambda: gemm.grouped_gemm(
            x, False, w1, True, gemm.EPI_PUSH, 0, bias=b1, heap_bases_ptr=blk.bases_ptr, heap_bases_host=blk.bases_host,
            push_data_off=blk.offset,
            push_flag_off=blk.offset + G * R * H * 2, push_rows=R, push_C=R, W=1, my_rank=0,
            budget_ms=tr.budget_ms, status_ptr=tr.status_ptr), args.iters, flush)
        report('gemm_push_local', ms, best, flops)
    if want('gemm_dgrad'):
        ms, best = timed(lambda: gemm.grouped_gemm(dy, False, w1, False, gemm.EPI_DACT, 2, aux=pre, out=out),
                         args.iters, flush)
        report('gemm_dgrad', ms, best, flops)
        traced('gemm_dgrad', lambda **kw: gemm.grouped_gemm(dy, False, w1, False, gemm.EPI_DACT, 2, aux=pre, out=out, **kw))
    if want('gemm_wgrad'):
        ms, best = timed(lambda: gemm.grouped_gemm(x, True, dy, True), args.iters, flush)
        report('gemm_wgrad', ms, best, flops)
        traced('gemm_wgrad', lambda **kw: gemm.grouped_gemm(x, True, dy, True, **kw))
    if want('cublas'):
        ms, best = timed(lambda: torch.bmm(x, w1, out=out), args.iters, flush)
        report('cublas_bmm', ms, best, flops)
        ms, best = timed(lambda: torch.bmm(x.transpose(1, 2), dy), args.iters, flush)
        report('cublas_bmm_wgrad', ms, best, flops)
    gemm.check_status()

    S, E, K = 8192, 2, 2
    C = K * (S // E)
    tok = torch.randn(S, M, device=dev).to(bf)
    logits = torch.randn(S, E, device=dev)
    idx, loc, gates, smap, top1, laux = lib.gate_forward(logits, K, C, True)
    if want('gate'):
        ms, best = timed(lambda: lib.gate_forward(logits, K, C, True), args.iters, flush)
        report('gate_forward', ms, best)
    if want('scatter'):
        ms, best = timed(lambda: lib.dispatch_scatter(tok, smap, None, K, E * C), args.iters, flush)
        report('dispatch_scatter', ms, best, bytes_=2.0 * E * C * M * 2)
    disp = lib.dispatch_scatter(tok, smap, None, K, E * C)
    if want('gather'):
        ms, best = timed(lambda: lib.dispatch_gather(disp, idx, loc, gates, C), args.iters, flush)
        report('dispatch_gather', ms, best, bytes_=(K + 1.0) * S * M * 2)
    if want('gate_grad'):
        ms, best = timed(lambda: lib.dispatch_gate_grad(disp, tok, idx, loc, C), args.iters, flush)
        report('gate_grad', ms, best, bytes_=(K + 1.0) * S * M * 2)
    if want('int8'):
        rows = disp[:8192]
        ms, best = timed(lambda: lib.int8_encode(rows), args.iters, flush)
        report('int8_encode', ms, best, bytes_=rows.numel() * 3.0)
        q, sc, bi = lib.int8_encode(rows)
        ms, best = timed(lambda: lib.int8_decode(q, sc, bi, bf), args.iters, flush)
        report('int8_decode', ms, best, bytes_=rows.numel() * 3.0)
    if want('colsum'):
        ms, best = timed(lambda: lib.colsum(dy), args.iters, flush)
        report('colsum', ms, best, bytes_=dy.numel() * 2.0)
        ms, best = timed(lambda: lib.colsum2(dy, x, 1, True), args.iters, flush)
        report('colsum2 (both bias gradients)', ms, best, bytes_=(dy.numel() + x.numel()) * 2.0)
    if want('misc'):
        import ctypes
        ms, best = timed(lambda: lib.int8_rows_encode(tok), args.iters, flush)
        report('int8_rows_encode', ms, best, bytes_=tok.numel() * 3.0)
        ms, best = timed(lambda: lib.importance_order(logits), args.iters, flush)
        report('importance_order', ms, best)
        rank, perm = lib.importance_order(logits)
        sm2 = smap.clone()
        ms, best = timed(lambda: lib.remap_slot_map(sm2, perm, K), args.iters, flush)
        report('remap_slot_map', ms, best)
        ms, best = timed(lambda: lib.build_slot_map(idx, loc, E, C), args.iters, flush)
        report('build_slot_map', ms, best)
        mask = (torch.rand(S, 16, device=dev) > 0.5).int()
        ms, best = timed(lambda: lib.cumsum_sub_one(mask), args.iters, flush)
        report('cumsum_sub_one', ms, best)
        flags = torch.ones(64, dtype=torch.int64, device=dev)
        st = gemm._status_word()
        ms, best = timed(lambda: lib.wait_flags(flags.data_ptr(), 64, 1, 100, st.device_ptr()), args.iters, flush)
        report('wait_flags(all set)', ms, best)
        ms, best = timed(lambda: lib.delay(20000), args.iters, flush)
        report('delay(20us)', ms, best)
        fn = ctypes.CDLL(lib.__file__).planmoe_colsum_bf16_noalloc
        fn.restype = ctypes.c_int
        fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_int, ctypes.c_longlong,
                       ctypes.c_longlong, ctypes.c_void_p]
        small = dy[:, :2048].contiguous()
        res = torch.empty(G, H, device=dev)
        stream = torch.cuda.current_stream().cuda_stream
        ms, best = timed(lambda: fn(small.data_ptr(), res.data_ptr(), G, small.size(1), H, small.stride(1), small.stride(0),
                                    stream), args.iters, flush)
        report('colsum_noalloc', ms, best, bytes_=small.numel() * 2.0)


if __name__ == '__main__':
    main()
