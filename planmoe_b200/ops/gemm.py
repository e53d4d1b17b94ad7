"""Python face of the tcgen05 grouped GEMM and the fused expert FFN built on it.

``grouped_gemm`` exposes the kernel of ``csrc/kernels/gemm_tcgen05.cu``: bf16 operands
``[groups, rows, cols]`` (optionally a leading split-K ``chunks`` dim), each either K-major or
MN-major, fp32 accumulation in TMEM, and one of four epilogues (store, bias+activation with the
activation's derivative saved, multiply by a saved derivative, push to peer ranks).

``expert_ffn`` is ``act(x @ W1 + b1) @ W2 + b2`` for all local experts with a hand-written
backward: six GEMM launches (2 forward, 2 dgrad, 2 wgrad) on the same kernel, activation and its
derivative fused into epilogues, bias gradients by a deterministic column-sum kernel.  It stands
in for the reference's two ``torch.matmul`` calls plus ATen bias/activation kernels and their
autograd (``PlanMoE/experts/ffn.py:63-82``).
"""

import torch

from . import native

import os

EPI_STORE, EPI_BIAS_ACT, EPI_DACT, EPI_PUSH = 0, 1, 2, 3
ACT_CODES = {'identity': 0, 'relu': 1, 'gelu': 2, 'silu': 3}

# CTA-group size used when a call does not name one: 0 lets the native launcher decide (two-CTA
# clusters unless a group has at most 128 rows, or PLANMOE_GEMM_CTA_GROUP overrides).
DEFAULT_CTA_GROUP = 0

_STATUS = None


def _status_word():
    """Process-wide status word for GEMMs launched outside a transport (local FFN, tests)."""
    global _STATUS
    if _STATUS is None:
        _STATUS = native.lib().StatusWord()
    return _STATUS


def check_status(sync=True):
    """Raise if a GEMM CTA gave up on a bounded wait since the last check."""
    if _STATUS is None:
        return
    if sync:
        torch.cuda.synchronize()
    st = _STATUS.read()
    if st[0] != 0:
        _STATUS.clear()
        raise RuntimeError("grouped GEMM: bounded wait expired, status %s" % (st[:4],))


def grouped_gemm(A, a_mn, B, b_mn, epilogue=EPI_STORE, activation=0, bias=None, aux=None, out=None,
                 **extra):
    """D[g] = A[g] . B[g].  ``a_mn`` / ``b_mn``: the operand's contiguous dim is its MN dim.

    A K-major: ``[G, M, K]``; A MN-major: ``[G, K, M]``; B K-major: ``[G, N, K]``; B MN-major:
    ``[G, K, N]``.  ``extra`` sets flag-gate / push / budget fields of ``GemmOpts``.
    """
    lib = native.lib()
    o = lib.GemmOpts()
    o.epilogue, o.activation = int(epilogue), int(activation)
    o.bias, o.aux, o.out = bias, aux, out
    o.cta_group = DEFAULT_CTA_GROUP
    for k, v in extra.items():
        setattr(o, k, v)
    if 'status_ptr' not in extra:
        o.status_ptr = _status_word().device_ptr()
    if 'budget_ms' not in extra:
        o.budget_ms = int(os.environ.get('PLANMOE_WAIT_BUDGET_MS', '20000'))
    return lib.grouped_gemm(A, bool(a_mn), B, bool(b_mn), o)


class _ExpertFFN(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w1, b1, w2, b2, act):
        x = x.contiguous()
        G, R, _ = x.shape
        H = w1.size(2)
        pre = torch.empty((G, R, H), dtype=x.dtype, device=x.device)
        h = grouped_gemm(x, False, w1, True, EPI_BIAS_ACT, act, bias=b1.contiguous(), aux=pre)
        y = grouped_gemm(h, False, w2, True, EPI_STORE, bias=b2.contiguous())
        ctx.save_for_backward(x, w1, w2, pre, h)
        ctx.act = act
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w1, w2, pre, h = ctx.saved_tensors
        dy = dy.contiguous()
        lib = native.lib()
        # dH_pre = (dY . W2^T) * act'(pre)        B = W2 [G, H, O]: N = H rows, K = O contiguous
        dh = grouped_gemm(dy, False, w2, False, EPI_DACT, ctx.act, aux=pre)
        # dX = dH_pre . W1^T                      B = W1 [G, M, H]: N = M rows, K = H contiguous
        dx = grouped_gemm(dh, False, w1, False, EPI_STORE)
        # dW2 = H^T . dY, dW1 = X^T . dH_pre      contraction over rows: both operands MN-major
        dw2 = grouped_gemm(h, True, dy, True, EPI_STORE)
        dw1 = grouped_gemm(x, True, dh, True, EPI_STORE)
        db2, db1 = lib.colsum2(dy, dh, 1, True)
        return dx, dw1, db1, dw2, db2, None


def expert_ffn(x, w1, b1, w2, b2, act_name):
    """x ``[E_local, rows, M]`` bf16 -> ``[E_local, rows, O]``."""
    return _ExpertFFN.apply(x, w1, b1, w2, b2, ACT_CODES[act_name])
