#!/usr/bin/env python3
"""End-to-end training throughput of the GPT-style MoE transformer on synthetic token ids.

    torchrun --nproc_per_node=8 -m planmoe_b200.examples.train_gpt_moe [--steps 20] [--layers 12] ...

Defaults: 12 layers, d_model 1024, 16 heads, seq 1024, vocab 32000, every other layer MoE with
8 experts per GPU (64 on 8 GPUs), FFN hidden 4096, top-2, capacity factor 1.25, global batch
64 sequences, bf16, AdamW.  Data parallel over sequences, expert parallel over the same ranks.
Prints one JSON line with tokens/s (CUDA events, max over ranks).
"""

import argparse
import json
import os

import torch
import torch.distributed as dist


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument('--steps', type=int, default=10)
    ap.add_argument('--warmup', type=int, default=3)
    ap.add_argument('--layers', type=int, default=12)
    ap.add_argument('--d_model', type=int, default=1024)
    ap.add_argument('--heads', type=int, default=16)
    ap.add_argument('--seq', type=int, default=1024)
    ap.add_argument('--vocab', type=int, default=32000)
    ap.add_argument('--ffn', type=int, default=4096)
    ap.add_argument('--experts_per_rank', type=int, default=8)
    ap.add_argument('--global_batch', type=int, default=64)
    ap.add_argument('--degree', default='1')
    ap.add_argument('--device', default='cuda' if torch.cuda.is_available() else 'cpu')
    ap.add_argument('--fused', type=int, default=1)
    args = ap.parse_args(argv)

    from planmoe_b200.models.gpt_moe import GPTMoE, GPTMoEConfig, allreduce_dense_grads

    world = int(os.environ.get('WORLD_SIZE', 1))
    rank = int(os.environ.get('RANK', 0))
    local = int(os.environ.get('LOCAL_RANK', 0))
    cuda = args.device == 'cuda'
    dev = torch.device('cuda', local) if cuda else torch.device('cpu')
    if cuda:
        torch.cuda.set_device(dev)
    if world > 1 and not dist.is_initialized():
        dist.init_process_group('nccl' if cuda else 'gloo', **({'device_id': dev} if cuda else {}))
    os.environ['PLANMOE_FUSED'] = str(args.fused)

    degree = args.degree if args.degree == 'auto' else int(args.degree)
    cfg = GPTMoEConfig(vocab_size=args.vocab, n_layer=args.layers, n_head=args.heads, d_model=args.d_model,
                       seq_len=args.seq, ffn_hidden=args.ffn, experts_per_rank=args.experts_per_rank, degree=degree)
    torch.manual_seed(1234)
    model = GPTMoE(cfg).to(dev)
    if cuda:
        model.cast_(torch.bfloat16)
    opt = torch.optim.AdamW(model.parameters(), lr=1e-4, fused=cuda)
    per_rank = max(1, args.global_batch // world)
    gen = torch.Generator(device='cpu').manual_seed(100 + rank)
    tokens = torch.randint(0, args.vocab, (per_rank, args.seq + 1), generator=gen).to(dev)

    def step():
        opt.zero_grad(set_to_none=True)
        loss = model(tokens[:, :-1], tokens[:, 1:])
        loss.backward()
        allreduce_dense_grads(model, None, world)
        opt.step()
        return loss

    def sync():
        if world > 1:
            dist.barrier()
        if cuda:
            torch.cuda.synchronize()

    losses = []
    for _ in range(args.warmup):
        losses.append(float(step()))
    sync()
    if cuda:
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
    else:
        import time
        t0 = time.perf_counter()
    for _ in range(args.steps):
        loss = step()
    if cuda:
        e.record()
        sync()
        ms = s.elapsed_time(e)
    else:
        ms = (time.perf_counter() - t0) * 1e3
    losses.append(float(loss))
    t = torch.tensor([ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if cuda:
        from planmoe_b200.parallel import transport
        transport.get_transport(None).check()
    if rank == 0:
        toks = per_rank * world * args.seq * args.steps
        print(json.dumps({'metric': 'gpt_moe_training_tokens_per_sec', 'value': toks / (float(t) / 1e3),
                          'ms_per_step': float(t) / args.steps, 'n_gpus': world, 'global_batch': per_rank * world,
                          'seq_len': args.seq, 'layers': args.layers, 'experts': args.experts_per_rank * world,
                          'first_loss': losses[0], 'last_loss': losses[-1], 'fused': args.fused}))
    return losses


if __name__ == '__main__':
    main()
    if dist.is_initialized():
        dist.destroy_process_group()
