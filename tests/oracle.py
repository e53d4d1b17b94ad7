"""Dense per-token reference of the MoE layer: y_t = sum_k g_{t,k} * FFN_{e_k}(x_t) with the
capacity drop rule, written with plain PyTorch ops only (no dispatch tensors)."""

import torch
import torch.nn.functional as F


def route_reference(scores, top_k, capacity_factor, normalize_gate=True, alignment=1):
    """Token-order slot assignment, python loops: (idx[k][t], loc[k][t], gate[k][t], capacity)."""
    S, E = scores.shape
    top_k = min(top_k, E)
    order = torch.topk(scores, top_k, dim=1).indices
    counts = [0] * E
    idx = [[0] * S for _ in range(top_k)]
    loc = [[0] * S for _ in range(top_k)]
    for k in range(top_k):
        for t in range(S):
            e = int(order[t, k])
            idx[k][t] = e
            loc[k][t] = counts[e]
            counts[e] += 1
    gates = scores.gather(1, order)
    if top_k > 1 and normalize_gate:
        gates = gates / torch.clamp(gates.sum(1, keepdim=True), min=torch.finfo(scores.dtype).eps)
    cap = top_k * int(capacity_factor * ((S + E - 1) // E))
    if cap % alignment:
        cap += alignment - cap % alignment
    return torch.tensor(idx), torch.tensor(loc), gates.t(), cap


def dense_moe_reference(x, wg, w1, b1, w2, b2, top_k, capacity_factor, act=F.relu,
                        normalize_gate=True, alignment=4, is_postscore=True):
    """x [S, M]; wg [E, M]; w1 [E, M, H]; b1 [E, H]; w2 [E, H, O]; b2 [E, O] (all experts)."""
    scores = F.softmax(x @ wg.t(), dim=1)
    idx, loc, gates, cap = route_reference(scores.detach(), top_k, capacity_factor, normalize_gate, alignment)
    gsel = scores.gather(1, idx.t())
    if top_k > 1 and normalize_gate:
        gsel = gsel / torch.clamp(gsel.sum(1, keepdim=True), min=torch.finfo(scores.dtype).eps)
    out = torch.zeros(x.size(0), w2.size(2), dtype=x.dtype)
    for k in range(idx.size(0)):
        keep = (loc[k] < cap)
        e = idx[k]
        g = gsel[:, k]
        xin = x if is_postscore else x * g[:, None]
        h = act(torch.einsum('tm,tmh->th', xin, w1[e]) + b1[e])
        y = torch.einsum('th,tho->to', h, w2[e]) + b2[e]
        if is_postscore:
            y = y * g[:, None]
        out = out + y * keep[:, None]
    S, E = scores.shape
    frac = torch.bincount(idx[0], minlength=E).to(scores.dtype) * (E / S)
    l_aux = (scores.sum(0) * frac).sum() / S
    return out, l_aux
