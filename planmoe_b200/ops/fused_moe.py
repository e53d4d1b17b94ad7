"""The fused expert-parallel MoE path for bf16 FFN experts on B200.

Forward, per pipeline chunk j of the capacity dimension (``degree`` chunks):

    fused gate kernel      softmax + top-k + slot scan + slot map + GShard loss
    dispatch + GEMM 1      ONE launch.  A copy warp in every CTA moves token rows (picked by slot
                           map) with the bulk-copy engine straight into the receive buffer of the
                           rank that owns the expert and release-adds its flag; the tcgen05 GEMM of
                           the same launch reads A tiles from its own receive buffer as soon as the
                           flags of the source ranks they touch have arrived; bias + activation
                           epilogue.  (With one rank a separate slot-major copy kernel runs first.)
    expert GEMM 2          tcgen05; the epilogue stores rows straight into the combine buffer of
                           the rank that owns the token, + release-add on its flag
    combine   (gather)     waits for the flags, gate-weighted sum over the k picks

Backward mirrors it (combine-backward is a dispatch-like push of dY, the two dgrad GEMMs are
flag-gated / pushing in the same way, dispatch-backward is a flag-waiting gather) and the two
weight-gradient GEMMs contract over all chunks of the receive buffers in one launch each.

No NCCL call and no library GEMM is on this path; with one rank the "peer" is the local heap and
the same kernels run.  The receive buffers are laid out ``[chunk][E_local][W_src][C/chunks][M]``,
i.e. they *are* the grouped-GEMM operands: the reference's permute copies, chunk splits and
concatenations (``PlanMoE/impls/overlap.py:55-75``, ``impls/communicate.py:604-623``) have no
counterpart here.

Buffer reuse: every layer owns a ring of buffer sets; a set is held from its forward until its
backward has run.  Two sets alternate in steady state — a peer can only write a set again after it
has passed the last exchange of the previous step, which every rank enters after its own reads.
Flags are never reset: each use adds a known number of arrivals, receivers wait for the
cumulative count.
"""

import os

import torch
import torch.nn.functional as F

from . import native
from .gemm import ACT_CODES, EPI_BIAS_ACT, EPI_DACT, EPI_PUSH, EPI_STORE, grouped_gemm
from ..parallel import transport as T
from ..utils.stage_timer import stage

MAX_CHUNKS = 32      # flag slots reserved per phase: [phase][chunk][source rank]
MAX_TOP_K = 4        # the fused gate kernel keeps at most four picks per token
PH_DISPATCH, PH_COMBINE, PH_COMBINE_BWD, PH_DISPATCH_BWD = 0, 1, 2, 3


class _BufferSet:
    """Symmetric receive buffers + flags for one in-flight forward/backward of one layer."""

    def __init__(self, tr, key):
        E_l, W, C, M, O = key[:5]
        self.tr = tr
        el = 2
        self.sz_x = E_l * W * C * M * el         # dispatch receive      [d][E_l][W][Cc][M]
        self.sz_y = E_l * W * C * O * el         # combine receive       [E_g][C][O]
        flags = 4 * MAX_CHUNKS * W * 8
        total = 2 * self.sz_x + 2 * self.sz_y + flags
        self.block = tr.alloc(total)
        self.off_x = self.block.offset
        self.off_y = self.off_x + self.sz_x
        self.off_dy = self.off_y + self.sz_y
        self.off_dx = self.off_dy + self.sz_y
        self.off_flags = self.off_dx + self.sz_x
        self.W = W
        # Cumulative arrivals expected on every flag of a phase.  The count lives in device memory and is
        # advanced by a tiny add kernel in stream order before each use, and the waiting kernels read it
        # from there: nothing about the step's history is baked into kernel arguments, so a captured
        # CUDA graph of a step can be replayed.
        self.want_dev = torch.zeros(4, dtype=torch.int64, device=tr.device)
        self.want_views = [self.want_dev[i:i + 1] for i in range(4)]
        self.bases_host = self.block.bases_host   # peers' base addresses, for tensor maps over their buffers
        self.held = False

    def off_of(self, phase):
        """Heap offset of the receive buffer the given phase writes."""
        return (self.off_x, self.off_y, self.off_dy, self.off_dx)[phase]

    def expect(self, phase, arrivals):
        """Every flag of ``phase`` will receive ``arrivals`` more; returns the device address of the new
        cumulative count (a u64)."""
        self.want_views[phase].add_(int(arrivals))
        return self.want_dev.data_ptr() + 8 * phase

    def flag_off(self, phase):
        return self.off_flags + phase * MAX_CHUNKS * self.W * 8

    def flag_ptr(self, phase, chunk=0):
        base = self.tr.segments[self.block.segment].local_base()
        return base + self.flag_off(phase) + chunk * self.W * 8

    def view(self, off, shape):
        return self.block.tensor(torch.bfloat16, shape, byte_offset=off - self.block.offset)


class FusedState:
    """Per-layer state of the fused path: transport handle and the ring of buffer sets."""

    def __init__(self, layer):
        self.tr = T.get_transport(layer.group)
        self.sets = {}
        self.turn = {}

    def acquire(self, key):
        ring = self.sets.setdefault(key, [])
        turn = self.turn.get(key, 0)
        if len(ring) < 2:
            ring.append(_BufferSet(self.tr, key))
            bs = ring[-1]
        else:
            bs = ring[turn % len(ring)]
            if bs.held:
                free = [b for b in ring if not b.held]
                if free:
                    bs = free[0]
                else:
                    ring.append(_BufferSet(self.tr, key))
                    bs = ring[-1]
        self.turn[key] = turn + 1
        bs.held = True
        return bs


_SM_COUNT = {}


def _sm_count():
    dev = torch.cuda.current_device()
    if dev not in _SM_COUNT:
        _SM_COUNT[dev] = int(torch.cuda.get_device_properties(dev).multi_processor_count)
    return _SM_COUNT[dev]


def _fuse_send(world):
    """Whether the dispatch send runs inside the flag-gated GEMM launch (a copy warp in every CTA, on the
    bulk-copy engine).
    With peers it does: transfer and math then overlap in one kernel.  With one rank nothing crosses
    NVLink and a separate copy kernel on the whole machine, run first, is the default; the environment
    variable PLANMOE_FUSE_SEND=0/1 overrides either way."""
    env = os.environ.get('PLANMOE_FUSE_SEND')
    if env is not None:
        return env not in ('0', '', 'false')
    return world > 1


def _send_and_gemm(lib, bs, phase, src, slot_map, gates, K, E, C, W, rank, d, grid, gemm):
    """Dispatch-style push of ``src`` plus the flag-gated GEMM that consumes it.  ``gemm(want_ptr, **copy)``
    enqueues the GEMM gated on the arrival count stored at ``want_ptr``; ``grid`` is its CTA count."""
    bases = bs.block.bases_ptr
    if not _fuse_send(W):
        ctas = 4 * _sm_count()
        lib.scatter_push(src, slot_map, gates, K, E, C, bases, bs.off_of(phase), bs.flag_off(phase), W, rank, d,
                         ctas, 0, d)
        gemm(bs.expect(phase, ctas))
    else:
        gemm(bs.expect(phase, grid), heap_bases_ptr=bases, copy_x=src, copy_slot_map=slot_map, copy_gates=gates,
             copy_K=K, copy_E_local=E // W, copy_C=C, copy_chunks=d, copy_ctas=grid,
             copy_data_off=bs.off_of(phase), copy_flag_off=bs.flag_off(phase))


class _Lease:
    """Returns a buffer set to its ring when the autograd node that holds it goes away, whether
    or not backward ever ran."""

    def __init__(self, bs):
        self.bs = bs

    def __del__(self):
        self.bs.held = False


class _FusedGate(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, top_k, capacity, normalize):
        lib = native.lib()
        logits = logits.contiguous()
        idx, loc, gates, slot_map, top1, l_aux = lib.gate_forward(logits, top_k, capacity, normalize)
        ctx.save_for_backward(logits, idx, top1)
        ctx.normalize = normalize
        ctx.mark_non_differentiable(idx, loc, slot_map)
        return gates, l_aux.view(()), idx, loc, slot_map

    @staticmethod
    def backward(ctx, dgates, dl_aux, *_):
        logits, idx, top1 = ctx.saved_tensors
        lib = native.lib()
        dg = dgates.contiguous().float() if dgates is not None else None
        dl = dl_aux.reshape(1).contiguous().float() if dl_aux is not None else None
        return lib.gate_backward(logits, idx, dg, dl, top1, ctx.normalize), None, None, None


def fused_gate(logits, top_k, capacity, normalize):
    """(gates [K,S] fp32, l_aux scalar fp32, idx, loc, slot_map) — differentiable in logits."""
    return _FusedGate.apply(logits, int(top_k), int(capacity), bool(normalize))


class _FusedExperts(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gates, w1, b1, w2, b2, meta):
        lib = native.lib()
        st, idx, loc, slot_map = meta['state'], meta['idx'], meta['loc'], meta['slot_map']
        tr = st.tr
        W, rank = tr.world, tr.rank
        E, C, d, K = meta['E'], meta['C'], meta['degree'], meta['K']
        E_l, Cc = E // W, C // d
        S, M = x.shape
        H, O = w1.size(2), w2.size(2)
        R = W * Cc                                  # rows per expert per chunk
        act = meta['act']
        postscore = meta['postscore']
        # Buffer sets are keyed by the pipeline degree as well: the flags of a set are cumulative counters
        # that advance together, chunk by chunk, only while every use has the same number of chunks.
        bs = st.acquire((E_l, W, C, M, O, d))
        bases = bs.block.bases_ptr
        budget, status = tr.budget_ms, tr.status_ptr
        gates_f = gates.detach().contiguous()

        # ---- dispatch + GEMM 1 ---------------------------------------------------------------------
        # The copy kernel stores my tokens into the experts' home ranks chunk by chunk; GEMM 1 covers all
        # chunks in one launch and starts a tile as soon as the flags of the (chunk, source) rows it reads
        # have arrived.  With more than one rank the two run concurrently.
        recv_x = bs.view(bs.off_x, (d * E_l, R, M))
        dact = torch.empty((d * E_l, R, H), dtype=x.dtype, device=x.device)
        h = torch.empty_like(dact)

        def gemm1(want_ptr, **copy):
            grouped_gemm(recv_x, False, w1, True, EPI_BIAS_ACT, act, bias=b1, aux=dact, out=h,
                         gate_flags_ptr=bs.flag_ptr(PH_DISPATCH, 0), gate_rows=Cc, gate_want_ptr=want_ptr,
                         chunk_groups=E_l, W=W, my_rank=rank, budget_ms=budget, status_ptr=status, **copy)
        with stage('fwd.dispatch+gemm1'):
            _send_and_gemm(lib, bs, PH_DISPATCH, x, slot_map, None if postscore else gates_f, K, E, C, W, rank, d,
                           lib.gemm_grid_ctas(d * E_l, R, H), gemm1)
        push_arrivals = lib.gemm_push_arrivals(E_l, R, O, Cc, rank)
        # GEMM 2 over all chunks: the epilogue pushes rows to the token owners' combine buffers
        with stage('fwd.gemm2+combine_push'):
            grouped_gemm(h, False, w2, True, EPI_PUSH, 0, bias=b2,
                         heap_bases_ptr=bases, heap_bases_host=bs.bases_host, push_data_off=bs.off_y,
                         push_flag_off=bs.flag_off(PH_COMBINE), push_rows=Cc, push_C=C,
                         chunk_groups=E_l, W=W, my_rank=rank, budget_ms=budget, status_ptr=status)
        want_y = bs.expect(PH_COMBINE, push_arrivals)

        # ---- combine: wait for every (chunk, expert rank) flag, gate-weighted sum over k ---------
        # flags of chunks 0..d-1 are consecutive: [d][W]
        with stage('fwd.combine_wait+decode'):
            out = lib.gather_wait(bs.block.local_ptr + (bs.off_y - bs.block.offset), x.dtype, O, idx, loc,
                                  gates_f if postscore else None, C, bs.flag_ptr(PH_COMBINE, 0), d * W, 0,
                                  budget, status, want_y)

        ctx.meta, ctx.bs = meta, bs
        ctx.save_for_backward(x, gates_f, w1, w2, dact, h)
        ctx.dims = (W, rank, E, C, d, K, E_l, Cc, S, M, H, O, R)
        ctx.lease = _Lease(bs)
        return out

    @staticmethod
    def backward(ctx, dout):
        lib = native.lib()
        meta, bs = ctx.meta, ctx.bs
        x, gates_f, w1, w2, dact, h = ctx.saved_tensors
        W, rank, E, C, d, K, E_l, Cc, S, M, H, O, R = ctx.dims
        st, idx, loc, slot_map = meta['state'], meta['idx'], meta['loc'], meta['slot_map']
        tr = st.tr
        act, postscore = meta['act'], meta['postscore']
        bases = bs.block.bases_ptr
        budget, status = tr.budget_ms, tr.status_ptr
        dout = dout.contiguous()

        recv_y = bs.view(bs.off_y, (E * C, O))
        dgates = None
        send_src, send_gates, send_K = dout, (gates_f if postscore else None), K
        if postscore and _fuse_send(W):
            # The fused send moves rows with the bulk-copy engine, which cannot scale them: the gate-gradient
            # pass, which reads every dY row anyway, also writes the gate-weighted copies (row = token * K + k,
            # the owner code of the slot map), and the send then moves those as they are.
            with stage('bwd.gate_grad'):
                dgates, send_src = lib.dispatch_gate_grad_scaled(recv_y, dout, idx, loc, gates_f, C)
            send_gates, send_K = None, 1
        elif postscore and ctx.needs_input_grad[1]:
            with stage('bwd.gate_grad'):
                dgates = lib.dispatch_gate_grad(recv_y, dout, idx, loc, C)

        # ---- combine backward: push dY (gate-weighted) + flag-gated dgrad 2 ---------------------------
        recv_dy = bs.view(bs.off_dy, (d * E_l, R, O))
        recv_x = bs.view(bs.off_x, (d * E_l, R, M))
        dh = torch.empty_like(dact)

        def dgrad2(want_ptr, **copy):
            # dH = (dY . W2^T) * act'
            grouped_gemm(recv_dy, False, w2, False, EPI_DACT, act, aux=dact, out=dh,
                         gate_flags_ptr=bs.flag_ptr(PH_COMBINE_BWD, 0), gate_rows=Cc, gate_want_ptr=want_ptr,
                         chunk_groups=E_l, W=W, my_rank=rank, budget_ms=budget, status_ptr=status, **copy)
        with stage('bwd.combine_bwd_send+dgrad2'):
            _send_and_gemm(lib, bs, PH_COMBINE_BWD, send_src, slot_map, send_gates, send_K, E, C, W, rank,
                           d, lib.gemm_grid_ctas(d * E_l, R, H), dgrad2)
        push_arrivals = lib.gemm_push_arrivals(E_l, R, M, Cc, rank)
        # dX slots = dH . W1^T, pushed back to the token owners
        with stage('bwd.dgrad1+dispatch_bwd_push'):
            grouped_gemm(dh, False, w1, False, EPI_PUSH, 0,
                         heap_bases_ptr=bases, heap_bases_host=bs.bases_host, push_data_off=bs.off_dx,
                         push_flag_off=bs.flag_off(PH_DISPATCH_BWD), push_rows=Cc, push_C=C,
                         chunk_groups=E_l, W=W, my_rank=rank, budget_ms=budget, status_ptr=status)
        want_dx = bs.expect(PH_DISPATCH_BWD, push_arrivals)

        # ---- weight / bias gradients: contract over all chunks in one launch each ---------------
        with stage('bwd.wgrad2'):
            dw2 = grouped_gemm(h.view(d, E_l, R, H), True, recv_dy.view(d, E_l, R, O), True, EPI_STORE)
        with stage('bwd.wgrad1'):
            dw1 = grouped_gemm(recv_x.view(d, E_l, R, M), True, dh.view(d, E_l, R, H), True, EPI_STORE)
        with stage('bwd.bias_grads'):
            db2 = lib.colsum(recv_dy, d, True)
            db1 = lib.colsum(dh, d, True)

        # ---- dispatch backward: wait for the returned slots, gather (gate-weighted if pre-score)
        with stage('bwd.dispatch_bwd_wait+gather'):
            dx = lib.gather_wait(bs.block.local_ptr + (bs.off_dx - bs.block.offset), dout.dtype, M, idx, loc,
                                 None if postscore else gates_f, C, bs.flag_ptr(PH_DISPATCH_BWD, 0), d * W,
                                 0, budget, status, want_dx)
        if not postscore and ctx.needs_input_grad[1]:
            recv_dx = bs.view(bs.off_dx, (E * C, M))
            dgates = lib.dispatch_gate_grad(recv_dx, x, idx, loc, C)
        return dx, dgates, dw1, db1, dw2, db2, None


def forward(layer, x, gctx, top_k, capacity_factor, degree):
    """Run the fused path for ``layer`` on tokens ``x [S, M]``; returns ``(y [S, O], l_aux)``."""
    if layer._fused is None:
        layer._fused = FusedState(layer)
    st = layer._fused
    S, M = x.shape
    E = layer.num_global_experts
    top_k = min(int(top_k), E)
    assert degree <= MAX_CHUNKS and top_k <= MAX_TOP_K, "plan outside the fused kernels' limits"

    with torch.autocast('cuda', enabled=False), stage('fwd.gate_linear'):
        logits = gctx(x)
        if layer.training and gctx.gate_noise > 0:
            logits = logits + gctx.gate_noise * torch.randn_like(logits) / E
    capacity = top_k * int(capacity_factor * ((S + E - 1) // E))
    align = 4 * layer.sharded_count * degree
    if capacity % align:
        capacity += align - capacity % align

    with stage('fwd.gate_topk_scan'):
        gates, l_aux, idx, loc, slot_map = fused_gate(logits, top_k, capacity, layer.normalize_gate)
    ex = layer.experts
    meta = dict(state=st, idx=idx, loc=loc, slot_map=slot_map, E=E, C=capacity, degree=degree, K=top_k,
                act=ACT_CODES[ex.act_name], postscore=layer.is_postscore)
    y = _FusedExperts.apply(x.contiguous(), gates, ex.batched_fc1_w, ex.batched_fc1_bias,
                            ex.batched_fc2_w, ex.batched_fc2_bias, meta)
    layer.last_stats = dict(capacity=capacity, degree=degree, path='fused')
    if getattr(layer, 'collect_stats', False):
        from ..utils import metrics
        layer.last_stats.update(metrics.routing_stats(idx, loc, E, capacity))
        layer.last_stats.update(metrics.wire_stats(E, capacity, M, x.element_size(), st.tr.world, layer.compress_name,
                                                   layer.comm_name, degree))
    return y, l_aux.to(logits.dtype)
