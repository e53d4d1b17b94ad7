"""Linear top-k gate: logits = x @ wg^T.

Reference: ``PlanMoE/gates/top.py:6-28``.  State-dict key ``wg.weight`` of shape
``[num_global_experts, model_dim]`` (fp32 when ``fp32_gate``).
"""

import torch
import torch.nn.functional as F

_ALLOWED = ('capacity_factor', 'gate_noise')


class LinearTopKGate(torch.nn.Module):
    def __init__(self, model_dim, num_global_experts, k=1, fp32_gate=False, **options):
        super().__init__()
        for opt in options:
            if opt not in _ALLOWED:
                raise Exception('Unrecognized argument provided to Gating module: %s' % opt)
        self.wg = torch.nn.Linear(model_dim, num_global_experts, bias=False,
                                  dtype=torch.float32 if fp32_gate else None)
        self.top_k = min(num_global_experts, int(k))
        self.fp32_gate = fp32_gate

    def forward(self, x):
        if self.fp32_gate:
            return F.linear(x.float(), self.wg.weight.float())
        return self.wg(x)


Gate = LinearTopKGate
