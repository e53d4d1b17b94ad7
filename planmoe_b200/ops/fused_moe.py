"""The fused expert-parallel MoE path for bf16 FFN experts on B200.

Forward, per pipeline chunk j of the capacity dimension (``degree`` chunks):

    fused gate kernel      softmax + top-k + slot scan + slot map + GShard loss
    dispatch + GEMM 1      ONE launch.  A copy warp in every CTA moves token rows (picked by slot
                           map) with the bulk-copy engine straight into the receive buffer of the
                           rank that owns the expert, eight rows at a time, and once their stores
                           have completed adds the row count to the flag of the 128-row block they
                           land in; the tcgen05 GEMM of the same launch reads a 128-row block of its
                           own receive buffer as soon as that block is complete; bias + activation
                           epilogue.  Transfer and math overlap 128 rows at a time, whatever the
                           pipeline degree.  With int8 rows a de-quantiser warp sits in between.
    expert GEMM 2          tcgen05; the epilogue stores rows straight into the combine buffer of
                           the rank that owns the token (bf16, or int8 with per-group scales), then
                           adds to its flag
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

MAX_CHUNKS = 32      # largest pipeline degree (flag slots per phase are sized for it)
MAX_TOP_K = 4        # the fused gate kernel keeps at most four picks per token
GATE_BLOCK = 128     # rows per arrival flag of a dispatched GEMM operand
MAX_ROW_BYTES = 16384  # longest bf16 row the fused send moves (one bulk-copy slot)
FUSED_CODECS = ('no', 'int8')  # wire formats of the fused kernels
# flag regions of a buffer set: the four exchanges, then the "de-quantised and ready" flags of the two
# dispatch-like exchanges when rows travel as int8
PH_DISPATCH, PH_COMBINE, PH_COMBINE_BWD, PH_DISPATCH_BWD, PH_DISPATCH_READY, PH_COMBINE_BWD_READY = range(6)
N_PHASES = 6


class _BufferSet:
    """Symmetric receive buffers + flags for one in-flight forward/backward of one layer."""

    def __init__(self, tr, key):
        E_l, W, C, M, O, d, q8 = key[:7]
        self.tr = tr
        rows = E_l * W * C
        self.q8 = bool(q8)
        self.sz_x = rows * M * 2                  # dispatch receive (bf16 GEMM operand)  [d][E_l][W][Cc][M]
        self.sz_dy = rows * O * 2                 # combine-backward receive (bf16 GEMM operand)
        if q8:
            self.sz_y = rows * (O + O // 16)      # combine receive, int8 rows + one (scale, low) per 128 columns
            self.sz_dx = rows * (M + M // 16)
            self.sz_qx = rows * (M + 16)          # int8 landing buffers of the two dispatch-like exchanges
            self.sz_qdy = rows * (O + 16)
        else:
            self.sz_y = rows * O * 2              # combine receive       [E_g][C][O]
            self.sz_dx = rows * M * 2
            self.sz_qx = self.sz_qdy = 0
        # flags of one phase: [chunk][source] arrivals (push epilogues, unfused send) or one row counter per
        # 128-row block of every (chunk, expert) group (fused send)
        self.flag_slots = max(MAX_CHUNKS * W, E_l * (W * C // GATE_BLOCK + MAX_CHUNKS) + 8)
        sizes = [self.sz_x, self.sz_y, self.sz_dy, self.sz_dx, self.sz_qx, self.sz_qdy, N_PHASES * self.flag_slots * 8]
        sizes = [(v + 1023) // 1024 * 1024 for v in sizes]
        self.block = tr.alloc(sum(sizes))
        offs = [self.block.offset]
        for v in sizes[:-1]:
            offs.append(offs[-1] + v)
        self.off_x, self.off_y, self.off_dy, self.off_dx, self.off_qx, self.off_qdy, self.off_flags = offs
        self.W = W
        # Cumulative arrivals expected on every flag of a phase.  The count lives in device memory and is
        # advanced by a tiny add kernel in stream order before each use, and the waiting kernels read it
        # from there: nothing about the step's history is baked into kernel arguments, so a captured
        # CUDA graph of a step can be replayed.
        self.want_dev = torch.zeros(N_PHASES, dtype=torch.int64, device=tr.device)
        self.want_views = [self.want_dev[i:i + 1] for i in range(N_PHASES)]
        self.bases_host = self.block.bases_host   # peers' base addresses, for tensor maps over their buffers
        self.held = False
        if T.debug_guards():
            # debug: receive buffers start as NaN (bf16) / 0xFF (int8 rows), so a slot that no sender wrote is
            # visible in the first step's output; the flags behind them stay zero
            data_bytes = self.off_flags - self.block.offset
            raw = self.block.tensor(torch.uint8, (data_bytes,))
            raw.fill_(0xFF)                            # 0xFFFF is a bf16 NaN
            if tr.world > 1 and not tr.emulated:
                torch.cuda.synchronize()
                import torch.distributed as dist
                dist.barrier(group=tr.group)           # nobody sends before every rank has finished poisoning

    def off_of(self, phase):
        """Heap offset of the bf16 receive buffer the given exchange fills."""
        return (self.off_x, self.off_y, self.off_dy, self.off_dx)[phase]

    def landing_off(self, phase):
        """Heap offset of the buffer peers store into for a dispatch-like exchange (the int8 landing buffer when
        rows travel as int8, else the bf16 operand itself)."""
        if self.q8:
            return self.off_qx if phase == PH_DISPATCH else self.off_qdy
        return self.off_of(phase)

    def expect(self, phase, arrivals):
        """Every flag of ``phase`` will receive ``arrivals`` more; returns the device address of the new
        cumulative count (a u64)."""
        self.want_views[phase].add_(int(arrivals))
        return self.want_dev.data_ptr() + 8 * phase

    def flag_off(self, phase):
        return self.off_flags + phase * self.flag_slots * 8

    def flag_ptr(self, phase, chunk=0):
        base = self.tr.segments[self.block.segment].local_base()
        return base + self.flag_off(phase) + chunk * self.W * 8

    def local_ptr(self, off):
        return self.block.local_ptr + (off - self.block.offset)

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
    bulk-copy engine): the default, with or without peers.  PLANMOE_FUSE_SEND=0 selects the separate
    slot-major copy kernel followed by the gated GEMM instead."""
    env = os.environ.get('PLANMOE_FUSE_SEND')
    if env is not None:
        return env not in ('0', '', 'false')
    return True


# Role trace of the fused launches (PLANMOE_GEMM_TRACE=1): per CTA, when the copy role ran and how long the TMA
# producer waited for rows; `last_trace()` summarises the most recent launch per exchange.
_TRACE = {}


def _local_first():
    """PLANMOE_LOCAL_FIRST=1: own rows are sent first and the tile loop starts on them.  Off by default: at 2 GPUs it
    measured 2.6 % slower per step (the first tile waits 15 us instead of 20, but the link idles while the own rows
    are copied and the second and third tiles then wait for the late remote rows)."""
    return 1 if os.environ.get('PLANMOE_LOCAL_FIRST', '0') == '1' else 0


def _trace_buffer(phase, device):
    if os.environ.get('PLANMOE_GEMM_TRACE', '0') != '1':
        return None
    if phase not in _TRACE:
        _TRACE[phase] = torch.zeros(256, 32, dtype=torch.int64, device=device)
    return _TRACE[phase]


def last_trace():
    """{exchange: {'kernel_us', 'copy_us', 'copy_start_us', 'gate_wait_us'}} medians / maxima over the CTAs."""
    out = {}
    for phase, buf in _TRACE.items():
        t = buf.cpu()
        t = t[t[:, 4] > 0]
        if t.numel() == 0:
            continue
        t0 = int(t[:, 0].min())
        out[{PH_DISPATCH: 'dispatch', PH_COMBINE_BWD: 'combine_bwd'}.get(phase, str(phase))] = {
            'kernel_us': (int(t[:, 4].max()) - t0) / 1e3,
            'copy_end_us_max': (int(t[:, 2].max()) - t0) / 1e3,
            'copy_end_us_median': (int(t[:, 2].median()) - t0) / 1e3,
            'copy_begin_us_median': (int(t[:, 1].median()) - t0) / 1e3,
            'gate_wait_us_median': float(t[:, 3].median()) / 1e3,
            'gate_wait_us_max': float(t[:, 3].max()) / 1e3,
            # per tile of a CTA's loop: when (after kernel entry) the producer asked for the rows, how long it waited
            'tile_ask_us_median': [round((int(t[:, 8 + 2 * i][t[:, 8 + 2 * i] > 0].median()) - t0) / 1e3, 1)
                                   for i in range(12) if bool((t[:, 8 + 2 * i] > 0).any())],
            'tile_wait_us_median': [round(float((t[:, 9 + 2 * i] - t[:, 8 + 2 * i])[t[:, 8 + 2 * i] > 0].median()) / 1e3, 1)
                                    for i in range(12) if bool((t[:, 8 + 2 * i] > 0).any())],
            'tile_wait_us_max': [round(float((t[:, 9 + 2 * i] - t[:, 8 + 2 * i])[t[:, 8 + 2 * i] > 0].max()) / 1e3, 1)
                                 for i in range(12) if bool((t[:, 8 + 2 * i] > 0).any())],
            'ctas': int(t.size(0))}
    return out


def _send_and_gemm(lib, bs, phase, src, slot_map, gates, K, E, C, W, rank, d, gemm):
    """Dispatch-style push of ``src`` plus the flag-gated GEMM that consumes it.  ``gemm(**gate_and_copy)``
    enqueues the GEMM with the given gate / copy / de-quantiser options."""
    bases = bs.block.bases_ptr
    Cc = C // d
    fused = _fuse_send(W) and gates is None and src.size(1) * src.element_size() <= MAX_ROW_BYTES
    if not fused:
        assert not bs.q8, "int8 rows travel only with the fused send"
        ctas = 4 * _sm_count()
        lib.scatter_push(src, slot_map, gates, K, E, C, bases, bs.off_of(phase), bs.flag_off(phase), W, rank, d,
                         ctas, 0, d)
        gemm(gate_flags_ptr=bs.flag_ptr(phase, 0), gate_rows=Cc, gate_want_ptr=bs.expect(phase, ctas))
        return
    nblk = (W * Cc + GATE_BLOCK - 1) // GATE_BLOCK
    opts = dict(gate_mode=1, gate_nblk=nblk, gate_want_ptr=bs.expect(phase, 1), perm_w=W, perm_seg_rows=Cc,
                perm_local_first=_local_first(),
                heap_bases_ptr=bases, copy_x=src, copy_slot_map=slot_map, copy_K=K, copy_E_local=E // W, copy_C=C,
                copy_chunks=d, copy_ctas=1, copy_data_off=bs.landing_off(phase), copy_flag_off=bs.flag_off(phase),
                copy_nblk=nblk)
    trace = _trace_buffer(phase, src.device)
    if trace is not None:
        opts['trace_ptr'] = trace.data_ptr()
    if bs.q8:
        ready = PH_DISPATCH_READY if phase == PH_DISPATCH else PH_COMBINE_BWD_READY
        opts.update(gate_flags_ptr=bs.flag_ptr(ready, 0), dq_ptr=bs.local_ptr(bs.landing_off(phase)),
                    dq_arrival_ptr=bs.flag_ptr(phase, 0), dq_ready_ptr=bs.flag_ptr(ready, 0))
    else:
        opts.update(gate_flags_ptr=bs.flag_ptr(phase, 0))
    gemm(**opts)


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
        q8 = bool(meta.get('q8', False))
        # ... and by the protocol of their flags: row counters per 128-row block (fused send) or one arrival per
        # sender CTA (separate copy kernel) must not be mixed on the same counters
        bs = st.acquire((E_l, W, C, M, O, d, q8, _fuse_send(W)))
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

        def gemm1(**gate):
            grouped_gemm(recv_x, False, w1, True, EPI_BIAS_ACT, act, bias=b1, aux=dact, out=h,
                         chunk_groups=E_l, W=W, my_rank=rank, budget_ms=budget, status_ptr=status, **gate)
        src = x
        if q8:
            # int8 wire: rows are quantised once per token (M bytes + a 16-byte scale trailer), the copy warps
            # move them as they are, and the de-quantiser warps of the receiving launch expand them in front of
            # the GEMM
            with stage('fwd.quantise'):
                src = lib.int8_rows_encode(x)
        with stage('fwd.dispatch+gemm1'):
            _send_and_gemm(lib, bs, PH_DISPATCH, src, slot_map, None if postscore else gates_f, K, E, C, W, rank, d,
                           gemm1)
        push_arrivals = lib.gemm_push_arrivals(E_l, R, O, Cc, rank)
        rows_y = E * C                              # rows of a combine buffer
        q8_push = dict(push_q8=1, push_scale_off=bs.off_y + rows_y * O) if q8 else {}
        # GEMM 2 over all chunks: the epilogue pushes rows to the token owners' combine buffers
        with stage('fwd.gemm2+combine_push'):
            grouped_gemm(h, False, w2, True, EPI_PUSH, 0, bias=b2,
                         heap_bases_ptr=bases, heap_bases_host=bs.bases_host, push_data_off=bs.off_y,
                         push_flag_off=bs.flag_off(PH_COMBINE), push_rows=Cc, push_C=C,
                         chunk_groups=E_l, W=W, my_rank=rank, budget_ms=budget, status_ptr=status, **q8_push)
        want_y = bs.expect(PH_COMBINE, push_arrivals)

        # ---- combine: wait for every (chunk, expert rank) flag, gate-weighted sum over k ---------
        # flags of chunks 0..d-1 are consecutive: [d][W]
        q8_gather = dict(q8_scales_ptr=bs.local_ptr(bs.off_y + rows_y * O), q8_group_rows=rows_y) if q8 else {}
        with stage('fwd.combine_wait+decode'):
            out = lib.gather_wait(bs.local_ptr(bs.off_y), x.dtype, O, idx, loc,
                                  gates_f if postscore else None, C, bs.flag_ptr(PH_COMBINE, 0), d * W, 0,
                                  budget, status, want_y, **q8_gather)

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

        q8 = bs.q8
        rows_y = E * C
        recv_y = None if q8 else bs.view(bs.off_y, (E * C, O))
        dgates = None
        send_src, send_gates, send_K = dout, (gates_f if postscore else None), K
        if q8:
            # expert outputs are held as int8 rows: the gate gradient de-quantises them on the fly; the gate-weighted
            # dY rows are quantised for the wire like the tokens were
            with stage('bwd.gate_grad'):
                dgates, send_src = lib.dispatch_gate_grad_q8(bs.local_ptr(bs.off_y), bs.local_ptr(bs.off_y + rows_y * O),
                                                             rows_y, dout, idx, loc, gates_f, C, True)
            send_gates, send_K = None, 1
        elif postscore and _fuse_send(W) and O * 2 <= MAX_ROW_BYTES:
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

        def dgrad2(**gate):
            # dH = (dY . W2^T) * act'
            grouped_gemm(recv_dy, False, w2, False, EPI_DACT, act, aux=dact, out=dh,
                         chunk_groups=E_l, W=W, my_rank=rank, budget_ms=budget, status_ptr=status, **gate)
        with stage('bwd.combine_bwd_send+dgrad2'):
            _send_and_gemm(lib, bs, PH_COMBINE_BWD, send_src, slot_map, send_gates, send_K, E, C, W, rank,
                           d, dgrad2)
        push_arrivals = lib.gemm_push_arrivals(E_l, R, M, Cc, rank)
        q8_push = dict(push_q8=1, push_scale_off=bs.off_dx + rows_y * M) if q8 else {}
        # dX slots = dH . W1^T, pushed back to the token owners
        with stage('bwd.dgrad1+dispatch_bwd_push'):
            grouped_gemm(dh, False, w1, False, EPI_PUSH, 0,
                         heap_bases_ptr=bases, heap_bases_host=bs.bases_host, push_data_off=bs.off_dx,
                         push_flag_off=bs.flag_off(PH_DISPATCH_BWD), push_rows=Cc, push_C=C,
                         chunk_groups=E_l, W=W, my_rank=rank, budget_ms=budget, status_ptr=status, **q8_push)
        want_dx = bs.expect(PH_DISPATCH_BWD, push_arrivals)

        # ---- weight / bias gradients: contract over all chunks in one launch each ---------------
        with stage('bwd.wgrad2'):
            dw2 = grouped_gemm(h.view(d, E_l, R, H), True, recv_dy.view(d, E_l, R, O), True, EPI_STORE)
        with stage('bwd.wgrad1'):
            dw1 = grouped_gemm(recv_x.view(d, E_l, R, M), True, dh.view(d, E_l, R, H), True, EPI_STORE)
        with stage('bwd.bias_grads'):
            db2, db1 = lib.colsum2(recv_dy, dh, d, True)

        # ---- dispatch backward: wait for the returned slots, gather (gate-weighted if pre-score)
        q8_gather = dict(q8_scales_ptr=bs.local_ptr(bs.off_dx + rows_y * M), q8_group_rows=rows_y) if q8 else {}
        with stage('bwd.dispatch_bwd_wait+gather'):
            dx = lib.gather_wait(bs.local_ptr(bs.off_dx), dout.dtype, M, idx, loc,
                                 None if postscore else gates_f, C, bs.flag_ptr(PH_DISPATCH_BWD, 0), d * W,
                                 0, budget, status, want_dx, **q8_gather)
        if not postscore and ctx.needs_input_grad[1]:
            recv_dx = bs.view(bs.off_dx, (E * C, M))
            dgates = lib.dispatch_gate_grad(recv_dx, x, idx, loc, C)
        return dx, dgates, dw1, db1, dw2, db2, None


def _dynamic_capacity(lib, logits, top_k, normalize, group, align):
    """Capacity for ``capacity_factor == 0``: the largest slot any expert hands out, over all ranks, plus one
    (reference: PlanMoE/impls/fast_dispatch.py:183-184, including its one host read of the all-reduced value).
    The value is rounded up to the next of a coarse ladder (steps of about 12 %) so that the buffer sets, which are
    keyed by capacity, take few distinct sizes; a larger capacity only adds empty slots."""
    with torch.no_grad():
        _idx, loc0, _g, _m, _t, _l = lib.gate_forward(logits.detach(), top_k, 4, normalize)
        peak = loc0.max().reshape(1).to(torch.int64)
        import torch.distributed as dist
        if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
            dist.all_reduce(peak, op=dist.ReduceOp.MAX, group=group)
        cap = int(peak.item()) + 1
    step = max(align, 64)
    ladder = step
    while ladder < cap:
        ladder = max(ladder + step, (int(ladder * 1.125) + step - 1) // step * step)
    return ladder


def check_routing_bounds(idx, loc, slot_map, S, E, capacity, top_k):
    """Bounds assertions on every index tensor the fused kernels address memory with (PLANMOE_DEBUG_GUARDS=1; costs
    host synchronisations).  ``idx [K, S]``: expert of each pick; ``loc [K, S]``: its slot (>= capacity = dropped);
    ``slot_map [E * capacity]``: owning pick ``token * K + k`` of each slot or -1.  Checked: ranges, that every kept
    pick owns exactly the slot that points back at it, and that no slot has two owners."""
    K = top_k
    assert idx.shape == (K, S) and loc.shape == (K, S) and slot_map.numel() == E * capacity, "routing tensor shapes"
    assert int(idx.min()) >= 0 and int(idx.max()) < E, "expert index out of range"
    assert int(loc.min()) >= 0, "negative slot"
    assert int(slot_map.min()) >= -1 and int(slot_map.max()) < S * K, "slot map entry out of range"
    kept = loc < capacity
    tok = torch.arange(S, device=idx.device).unsqueeze(0).expand(K, S)
    kk = torch.arange(K, device=idx.device).unsqueeze(1).expand(K, S)
    slots = (idx.long() * capacity + loc.long())[kept]
    owners = (tok * K + kk)[kept]
    assert torch.equal(slot_map.long()[slots], owners), "a kept pick does not own its slot"
    assert int((slot_map >= 0).sum()) == int(kept.sum()), "slot map has owners that no pick claims"


def forward(layer, x, gctx, top_k, capacity_factor, degree):
    """Run the fused path for ``layer`` on tokens ``x [S, M]``; returns ``(y [S, O], l_aux)``.

    Routing variants of the reference, all on the fused gate kernels: ``capacity_factor < 0`` uses its bound
    ``top_k * int(-cf * ceil(S / E))`` as the capacity (the reference takes the smaller of that bound and the largest
    slot in use, PlanMoE/impls/fast_dispatch.py:185-186; the same tokens are kept either way and no host read is
    needed); ``capacity_factor == 0`` sizes the capacity to the largest slot in use (one host read, as in the
    reference); batch-prioritised routing scans the slots in the order of the tokens' best scores (a counting-rank
    kernel, then the same gate kernels on the reordered logits); the load-importance loss replaces the GShard loss
    when ``is_gshard_loss`` is false (a few element-wise operations on the [S, E] scores)."""
    lib = native.lib()
    if layer._fused is None:
        layer._fused = FusedState(layer)
    st = layer._fused
    S, M = x.shape
    E = layer.num_global_experts
    top_k = min(int(top_k), E)
    assert degree <= MAX_CHUNKS and top_k <= MAX_TOP_K, "plan outside the fused kernels' limits"

    with torch.autocast('cuda', enabled=False), stage('fwd.gate_linear'):
        clean = gctx(x)
        logits = clean
        if layer.training and gctx.gate_noise > 0:
            logits = clean + gctx.gate_noise * torch.randn_like(clean) / E
        logits = logits.contiguous()
    align = 4 * layer.sharded_count * degree
    per_expert = (S + E - 1) // E
    if capacity_factor > 0:
        capacity = top_k * int(capacity_factor * per_expert)
    elif capacity_factor < 0:
        capacity = top_k * int(-capacity_factor * per_expert)
    else:
        capacity = _dynamic_capacity(lib, logits, top_k, layer.normalize_gate, layer.group, align)
    capacity = max(capacity, 1)
    if capacity % align:
        capacity += align - capacity % align

    with stage('fwd.gate_topk_scan'):
        if layer.batch_prioritized_routing:
            rank, perm = lib.importance_order(logits.detach())
            gates_p, l_aux, idx_p, loc_p, slot_map = fused_gate(logits.index_select(0, perm.long()), top_k, capacity,
                                                                layer.normalize_gate)
            pos = rank.long()
            gates = gates_p.index_select(1, pos)
            idx, loc = idx_p.index_select(1, pos).contiguous(), loc_p.index_select(1, pos).contiguous()
            lib.remap_slot_map(slot_map, perm, top_k)
        else:
            gates, l_aux, idx, loc, slot_map = fused_gate(logits, top_k, capacity, layer.normalize_gate)
    if not layer.is_gshard_loss:
        from ..impls import losses
        topk_logits = logits.float().gather(1, idx.t().long())
        l_aux = losses.load_importance_loss(F.softmax(clean.float(), dim=1), topk_logits, E, gctx.gate_noise)
    if T.debug_guards():
        check_routing_bounds(idx, loc, slot_map, S, E, capacity, top_k)
    ex = layer.experts
    meta = dict(state=st, idx=idx, loc=loc, slot_map=slot_map, E=E, C=capacity, degree=degree, K=top_k,
                act=ACT_CODES[ex.act_name], postscore=layer.is_postscore, q8=(layer.compress_name == 'int8'))
    y = _FusedExperts.apply(x.contiguous(), gates, ex.batched_fc1_w, ex.batched_fc1_bias,
                            ex.batched_fc2_w, ex.batched_fc2_bias, meta)
    # both 'naive' and 'pipe' run as the flat push of the copy role / push epilogue: say so instead of echoing the name
    layer.last_stats = dict(capacity=capacity, degree=degree, path='fused', comm='flat-push',
                            wire=('int8' if meta['q8'] else 'bf16'))
    if getattr(layer, 'collect_stats', False):
        from ..utils import metrics
        layer.last_stats.update(metrics.routing_stats(idx, loc, E, capacity))
        layer.last_stats.update(metrics.wire_stats(E, capacity, M, x.element_size(), st.tr.world, layer.compress_name,
                                                   layer.comm_name, degree))
    return y, l_aux.to(logits.dtype)
