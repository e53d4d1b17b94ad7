#!/usr/bin/env python3
"""Codec kernels on expert activations: throughput, compression ratio and error on one GPU.

    python -m planmoe_b200.examples.codec_bench [--rows 8192] [--cols 4096] [--iters 10]

Input: ``[rows, cols]`` bf16 taken as ReLU(N(0,1)), so about half of the values are exact zeros
(the shape of an expert's hidden activations).  Codecs: ``int8`` (row-affine 8 bit), ``zfp``
(fixed rate, 8 bits per value, 4 x 4 blocks) and ``lz`` (lossless, 16-bit symbols).  For every codec
the encode and the decode kernels are timed with CUDA events (L2 flushed by a 256 MiB write before
each launch, best and mean of ``--iters``); GB/s is quoted on the raw bf16 bytes for encode + decode
together, ratio = raw bytes / wire bytes, error = max |decoded - input|.  One JSON line per codec.
The reference's counterparts are ``PlanMoE/custom/compressor/{int8,zfpc,lz}.cpp`` and ``gpulz.cu``.
"""

import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument('--rows', type=int, default=8192)
    ap.add_argument('--cols', type=int, default=4096)
    ap.add_argument('--iters', type=int, default=10)
    ap.add_argument('--codecs', default='int8,zfp,lz')
    ap.add_argument('--world', type=int, default=8, help='destination slices the tensor is split into')
    args = ap.parse_args(argv)

    from planmoe_b200.parallel import codecs
    dev = 'cuda'
    torch.manual_seed(0)
    x = torch.relu(torch.randn(args.rows, args.cols, device=dev)).to(torch.bfloat16)
    x3 = x.view(args.world, -1, args.cols)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    raw = x.numel() * 2
    hbm = 6540.8
    peaks = os.path.join(ROOT, 'MEASURED_PEAKS.json')
    if os.path.exists(peaks):
        hbm = json.load(open(peaks))['hbm_gbs']

    def timed(fn):
        for _ in range(3):
            r = fn()
        torch.cuda.synchronize()
        best, total = 1e9, 0.0
        for i in range(args.iters):
            flush.fill_(i & 0xff)
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            r = fn()
            e.record()
            e.synchronize()
            ms = s.elapsed_time(e)
            best, total = min(best, ms), total + ms
        return r, best, total / args.iters

    for name in args.codecs.split(','):
        comp = codecs.get_compressor(name)
        packed, enc_best, enc_mean = timed(lambda: comp.compress(x3, args.world))
        out, dec_best, dec_mean = timed(lambda: comp.decompress(packed))
        err = (out.float().view_as(x) - x.float()).abs().max().item()
        wire = packed.wire_bytes()
        print(json.dumps({
            'case': 'codec', 'codec': name, 'rows': args.rows, 'cols': args.cols, 'zeros_frac': round((x == 0).float().mean().item(), 3),
            'encode_ms': round(enc_best, 4), 'decode_ms': round(dec_best, 4),
            'encode_ms_mean': round(enc_mean, 4), 'decode_ms_mean': round(dec_mean, 4),
            'raw_gbs_encode_plus_decode': round(2 * raw / ((enc_best + dec_best) * 1e-3) / 1e9, 1),
            'raw_gbs_encode': round(raw / (enc_best * 1e-3) / 1e9, 1),
            'raw_gbs_decode': round(raw / (dec_best * 1e-3) / 1e9, 1),
            'of_measured_hbm_encode': round((raw + wire) / (enc_best * 1e-3) / 1e9 / hbm, 3),
            'ratio': round(raw / wire, 3), 'wire_bytes': int(wire), 'max_abs_err': err,
            'lossless': bool(err == 0.0)}), flush=True)


if __name__ == '__main__':
    main()
