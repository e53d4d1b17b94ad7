"""Cosine-similarity top-k gate.

Reference: ``PlanMoE/gates/cosine_top.py:7-36``.  logits = normalize(proj(x)) .
normalize(sim_matrix) * exp(min(temperature, log 100)).  State-dict keys: ``temperature`` [1],
``cosine_projector.{weight,bias}`` ([proj_dim, M], [proj_dim]), ``sim_matrix`` [proj_dim, E].
"""

import math
import torch
import torch.nn.functional as F

_ALLOWED = ('capacity_factor', 'gate_noise')
_MAX_LOG_SCALE = math.log(1.0 / 0.01)


class CosineTopKGate(torch.nn.Module):
    def __init__(self, model_dim, num_global_experts, k=1, fp32_gate=False, proj_dim=256,
                 init_t=0.5, **options):
        super().__init__()
        for opt in options:
            if opt not in _ALLOWED:
                raise Exception('Unrecognized argument provided to Gating module: %s' % opt)
        self.top_k = min(num_global_experts, int(k))
        self.fp32_gate = fp32_gate
        self.temperature = torch.nn.Parameter(torch.log(torch.full([1], 1.0 / init_t)))
        self.cosine_projector = torch.nn.Linear(model_dim, proj_dim)
        self.sim_matrix = torch.nn.Parameter(torch.randn(size=(proj_dim, num_global_experts)))
        torch.nn.init.normal_(self.sim_matrix, 0, 0.01)

    def forward(self, x):
        w, b, sim = self.cosine_projector.weight, self.cosine_projector.bias, self.sim_matrix
        if self.fp32_gate:
            x, w, b, sim = x.float(), w.float(), b.float(), sim.float()
        proj = F.normalize(F.linear(x, w, b), dim=1)
        logits = proj @ F.normalize(sim, dim=0)
        scale = torch.clamp(self.temperature, max=_MAX_LOG_SCALE).exp()
        return logits * scale.to(logits.dtype)


Gate = CosineTopKGate
