"""GPT-style decoder with Mixture-of-Experts feed-forward layers.

The reference ships no model of its own; it patches Megatron-LM and fairseq so that decoder MLPs
become ``moe_layer`` (``PlanMoE/examples/megatron/schemoe_megatron.diff:54-101``,
``examples/fairseq_moe/fairseq_patch.diff:41-54``).  This module is the in-repo equivalent used for
end-to-end training throughput: pre-LN transformer blocks, causal self-attention through PyTorch's
fused scaled-dot-product attention, and every ``moe_every``-th block's MLP replaced by the
expert-parallel ``moe_layer`` (fused sm_100a path on CUDA).  Experts are sharded over the ranks
(expert parallel); everything else is replicated (data parallel) and marked for gradient
all-reduce by ``dense_parameters()``.
"""

import math
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..impls.moe_layer import moe_layer


@dataclass
class GPTMoEConfig:
    vocab_size: int = 32000
    n_layer: int = 12
    n_head: int = 16
    d_model: int = 1024
    seq_len: int = 1024
    ffn_hidden: int = 4096
    moe_every: int = 2              # every moe_every-th layer is MoE (0 = dense model)
    experts_per_rank: int = 8
    top_k: int = 2
    capacity_factor: float = 1.25
    aux_weight: float = 0.01
    degree: object = 1              # a2a_ffn_overlap_degree: int or 'auto'
    compress_name: str = 'no'
    comm_name: str = 'naive'
    fp32_gate: bool = True
    activation: str = 'gelu'


class CausalSelfAttention(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        self.n_head = cfg.n_head
        self.qkv = nn.Linear(cfg.d_model, 3 * cfg.d_model)
        self.proj = nn.Linear(cfg.d_model, cfg.d_model)

    def forward(self, x):
        B, T, D = x.shape
        q, k, v = self.qkv(x).view(B, T, 3, self.n_head, D // self.n_head).permute(2, 0, 3, 1, 4)
        y = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        return self.proj(y.transpose(1, 2).reshape(B, T, D))


class DenseMLP(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        self.fc1 = nn.Linear(cfg.d_model, cfg.ffn_hidden)
        self.fc2 = nn.Linear(cfg.ffn_hidden, cfg.d_model)

    def forward(self, x):
        y = self.fc2(F.gelu(self.fc1(x)))
        y.l_aux = None
        return y


class Block(nn.Module):
    def __init__(self, cfg, use_moe, group, layer_index):
        super().__init__()
        self.ln1 = nn.LayerNorm(cfg.d_model)
        self.attn = CausalSelfAttention(cfg)
        self.ln2 = nn.LayerNorm(cfg.d_model)
        if use_moe:
            self.mlp = moe_layer(
                gate_type={'type': 'top', 'k': cfg.top_k, 'capacity_factor': cfg.capacity_factor,
                           'fp32_gate': cfg.fp32_gate},
                model_dim=cfg.d_model,
                experts={'type': 'ffn', 'count_per_node': cfg.experts_per_rank,
                         'hidden_size_per_expert': cfg.ffn_hidden, 'activation_fn': cfg.activation},
                group=group, a2a_ffn_overlap_degree=cfg.degree, compress_name=cfg.compress_name,
                comm_name=cfg.comm_name, index=layer_index,
                scan_expert_func=lambda name, p: setattr(p, 'allreduce', False))
        else:
            self.mlp = DenseMLP(cfg)
        self.is_moe = use_moe

    def forward(self, x):
        x = x + self.attn(self.ln1(x))
        y = self.mlp(self.ln2(x))
        return x + y, getattr(y, 'l_aux', None)


class GPTMoE(nn.Module):
    def __init__(self, cfg, group=None):
        super().__init__()
        self.cfg = cfg
        self.tok = nn.Embedding(cfg.vocab_size, cfg.d_model)
        self.pos = nn.Embedding(cfg.seq_len, cfg.d_model)
        self.blocks = nn.ModuleList([
            Block(cfg, cfg.moe_every > 0 and (i % cfg.moe_every == cfg.moe_every - 1), group, i)
            for i in range(cfg.n_layer)])
        self.ln_f = nn.LayerNorm(cfg.d_model)
        self.apply(self._init)

    @staticmethod
    def _init(m):
        if isinstance(m, nn.Linear):
            nn.init.normal_(m.weight, std=0.02)
            if m.bias is not None:
                nn.init.zeros_(m.bias)
        elif isinstance(m, nn.Embedding):
            nn.init.normal_(m.weight, std=0.02)

    def cast_(self, dtype):
        """Cast to ``dtype`` but keep fp32 gates in fp32."""
        self.to(dtype)
        if self.cfg.fp32_gate:
            for b in self.blocks:
                if b.is_moe:
                    for g in b.mlp.gates:
                        g.float()
        return self

    def dense_parameters(self):
        """Replicated parameters (to be all-reduced over the data-parallel ranks)."""
        return [p for p in self.parameters() if not hasattr(p, '_tutel_expert')]

    def expert_parameters(self):
        return [p for p in self.parameters() if hasattr(p, '_tutel_expert')]

    def forward(self, tokens, targets=None):
        B, T = tokens.shape
        pos = torch.arange(T, device=tokens.device)
        x = self.tok(tokens) + self.pos(pos)
        aux = None
        for blk in self.blocks:
            x, l_aux = blk(x)
            if l_aux is not None:
                aux = l_aux.float() if aux is None else aux + l_aux.float()
        x = self.ln_f(x)
        logits = F.linear(x, self.tok.weight)
        if targets is None:
            return logits
        loss = F.cross_entropy(logits.float().view(-1, logits.size(-1)), targets.reshape(-1))
        if aux is not None:
            loss = loss + self.cfg.aux_weight * aux
        return loss


def allreduce_dense_grads(model, group=None, world_size=1, bucket_mb=64):
    """Average the replicated parameters' gradients over the ranks with a few large NCCL all-reduces
    (NVSwitch cost is per launch, not per link: buckets are sized for launch latency)."""
    import torch.distributed as dist
    if world_size <= 1:
        return
    params = [p for p in model.dense_parameters() if p.grad is not None]
    bucket, size = [], 0
    limit = bucket_mb << 20

    def flush():
        nonlocal bucket, size
        if not bucket:
            return
        flat = torch.cat([p.grad.reshape(-1) for p in bucket])
        dist.all_reduce(flat, group=group)
        flat.div_(world_size)
        off = 0
        for p in bucket:
            n = p.grad.numel()
            p.grad.copy_(flat[off:off + n].view_as(p.grad))
            off += n
        bucket, size = [], 0

    by_dtype = {}
    for p in params:
        by_dtype.setdefault(p.grad.dtype, []).append(p)
    for plist in by_dtype.values():
        for p in plist:
            bucket.append(p)
            size += p.grad.numel() * p.grad.element_size()
            if size >= limit:
                flush()
        flush()
