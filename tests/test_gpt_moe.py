"""GPT-MoE model: a tiny CPU training run must reduce the loss; parameter partition into replicated
and expert parameters; GPU smoke of the fused path inside the model."""

import pytest
import torch


def test_tiny_gpt_moe_trains_on_cpu():
    from planmoe_b200.models.gpt_moe import GPTMoE, GPTMoEConfig
    torch.manual_seed(0)
    cfg = GPTMoEConfig(vocab_size=64, n_layer=2, n_head=2, d_model=32, seq_len=16, ffn_hidden=64,
                       experts_per_rank=4, top_k=2, capacity_factor=2.0)
    model = GPTMoE(cfg)
    assert len(model.expert_parameters()) == 4 and len(model.dense_parameters()) > 8
    assert all(getattr(p, 'allreduce', True) is False for p in model.expert_parameters())
    opt = torch.optim.AdamW(model.parameters(), lr=3e-3)
    toks = torch.randint(0, 64, (4, 17))
    first = last = None
    for i in range(30):
        opt.zero_grad()
        loss = model(toks[:, :-1], toks[:, 1:])
        loss.backward()
        opt.step()
        first = float(loss) if first is None else first
        last = float(loss)
    assert last < first * 0.8, (first, last)


def test_train_example_cpu():
    from planmoe_b200.examples import train_gpt_moe
    losses = train_gpt_moe.main(['--device', 'cpu', '--steps', '2', '--warmup', '1', '--layers', '2', '--d_model', '32',
                                 '--heads', '2', '--seq', '16', '--vocab', '64', '--ffn', '64',
                                 '--experts_per_rank', '2', '--global_batch', '2'])
    assert all(l == l for l in losses)


@pytest.mark.gpu
def test_gpt_moe_fused_path_on_gpu():
    from planmoe_b200.models.gpt_moe import GPTMoE, GPTMoEConfig
    torch.manual_seed(0)
    cfg = GPTMoEConfig(vocab_size=512, n_layer=2, n_head=4, d_model=256, seq_len=128, ffn_hidden=512,
                       experts_per_rank=4)
    model = GPTMoE(cfg).cuda().cast_(torch.bfloat16)
    toks = torch.randint(0, 512, (8, 129), device='cuda')
    opt = torch.optim.AdamW(model.parameters(), lr=1e-3, fused=True)
    losses = []
    for _ in range(8):
        opt.zero_grad()
        loss = model(toks[:, :-1], toks[:, 1:])
        loss.backward()
        opt.step()
        losses.append(float(loss))
    assert model.blocks[1].mlp.last_stats['path'] == 'fused'
    assert losses[-1] < losses[0]
    from planmoe_b200.parallel import transport
    transport.get_transport(None).check()
