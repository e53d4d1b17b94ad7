"""Auxiliary load-balancing losses of the MoE gate.

Behavioural parity with the reference's ``PlanMoE/impls/losses.py:7-42``:
``gshard_loss`` (GShard / Switch balance loss on the top-1 assignment) and
``load_importance_loss`` (CV^2 of importance plus CV^2 of the Normal-CDF load).
"""

import torch


def _one_hot_with_dtype(data, num_classes, dtype, hot_value=1):
    """[N] integer class ids -> [N, num_classes] one-hot of ``dtype`` holding ``hot_value``."""
    out = torch.zeros((data.size(0), num_classes), device=data.device, dtype=dtype)
    return out.scatter_(1, data.reshape(-1, 1).long(), hot_value)


def gshard_loss(scores_w_noise, top_ids):
    """E * sum_e( mean_t score[t,e] * fraction of tokens whose top-1 expert is e ).

    ``top_ids`` is ``[S, k]``; only column 0 (the top-1 pick) enters the loss.
    """
    num_samples, num_experts = int(scores_w_noise.size(0)), int(scores_w_noise.size(1))
    top1 = top_ids[:, 0].long()
    frac = torch.bincount(top1, minlength=num_experts).to(scores_w_noise.dtype)
    frac = frac * (num_experts / num_samples)
    mean_score = scores_w_noise.sum(dim=0)
    return (mean_score * frac).sum() / num_samples


def _cv_squared(v):
    v = v.float()
    return v.var() / (v.mean() ** 2 + 1e-10)


def load_importance_loss(scores_wo_noise, topk_logits, num_global_experts, gate_noise):
    """0.5 * (CV^2(importance) + CV^2(load)), load estimated through a Normal CDF whose
    standard deviation is ``gate_noise / num_global_experts``."""
    importance = scores_wo_noise.float().sum(0)
    l_imp = _cv_squared(importance)

    std = max(float(gate_noise) / num_global_experts, 1e-20)
    threshold = topk_logits[:, -1].reshape(-1, 1).float()
    z = (scores_wo_noise.float() - threshold) / std
    prob = 0.5 * (1.0 + torch.erf(z * 0.7071067811865476))
    l_load = _cv_squared(prob.sum(0))
    return (l_imp + l_load) / 2.0
