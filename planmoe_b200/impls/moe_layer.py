"""The Mixture-of-Experts layer (``moe_layer``).

Public contract of the reference's ``PlanMoE/impls/moe_layer.py:27-314``: constructor keywords
(:44-64, unknown ones raise :73-75), ``forward(input, gate_index, capacity_factor, top_k,
a2a_ffn_overlap_degree, reserve_dims)`` (:213), output of the input's shape and dtype carrying
``.l_aux``, ``get_parameter_iterator``, expert-parameter tagging ``_tutel_expert``, env
switches ``SKIP_MOE`` / ``BATCH_PRIO`` / ``CAP_FACTOR``, and the state_dict keys
``gates.{i}.*`` / ``experts.batched_fc{1,2}_{w,bias}``.

Two execution paths:
  * fused (CUDA, bf16 FFN experts, linear top-k gate with the GShard loss): the sm_100a kernels in
    ``planmoe_b200.ops.fused_moe`` — fused gate, dispatch that stores into peer GPUs' receive
    buffers, flag-gated tcgen05 expert GEMMs, combine pushed back from the GEMM epilogue;
  * generic (everything else, CPU included): encode -> chunked codec/all-to-all/expert pipeline
    (``impls.overlap``) -> decode.

``a2a_ffn_overlap_degree`` may be an int (fixed chunk count, as in the reference) or
``'auto'`` / 0, and ``comm_name`` may be ``'auto'``: the adaptive scheduler
(``planmoe_b200.parallel.scheduler``) then calibrates once at the first forward (device-timed
repetitions of this layer's own forward + backward) and freezes one plan for all ranks.

Sharded experts (fewer experts than ranks) work in both modes the reference declares but
cannot run: ``parallel_type='model'`` splits the hidden dimension and sums partial outputs,
``'data'`` splits an expert's slots over its shard ranks and gathers the weights.
"""

import importlib
import logging
import os
import re

import torch
import torch.distributed as dist
import torch.nn.functional as F
from torch.nn import ModuleList

from . import communicate as C
from . import losses
from .fast_dispatch import extract_critical, fast_decode, fast_encode
from .overlap import a2a_ffn_overlap_forward

_NAME_RE = re.compile(r'^[a-zA-Z0-9_]+$')


def fused_codecs():
    """Codecs the fused kernels carry on the wire themselves."""
    from ..ops import fused_moe
    return fused_moe.FUSED_CODECS


def _import_builtin(kind, name):
    assert _NAME_RE.match(name), \
        "%s type must only include digits, letters and underline characters." % kind.capitalize()
    try:
        return importlib.import_module('planmoe_b200.%ss.%s' % (kind, name))
    except ModuleNotFoundError:
        raise Exception('Builtin %s type is not recognized: %s' % (kind, name))


class MOELayer(torch.nn.Module):

    @staticmethod
    def global_expert_count(num_local_experts, group=None):
        """``count_per_node`` > 0: experts per rank; < 0: ranks per expert; a fraction 1/n
        means n ranks share one expert."""
        if not isinstance(num_local_experts, int):
            num_local_experts = -int(1 / (num_local_experts + 1e-5))
        world_size = C.get_world_size(group)
        if num_local_experts == 0:
            raise Exception("Invalid value of num_local_experts: %d" % num_local_experts)
        if num_local_experts > 0:
            return num_local_experts * world_size
        assert world_size % -num_local_experts == 0, \
            "Excepting %d devices to share an expert param, while global device count is %d." % (
                -num_local_experts, world_size)
        return world_size // -num_local_experts

    def __init__(self, gate_type, model_dim, experts=None, scan_expert_func=None,
                 result_func=None, group=None, seeds=None, a2a_ffn_overlap_degree=1,
                 is_postscore=True, batch_prioritized_routing=False, normalize_gate=True,
                 is_gshard_loss=True, parallel_type='auto', use_2dh=False, index=0,
                 compress_name='no', comm_name='naive', **kwargs):
        super().__init__()
        assert model_dim % 2 == 0, \
            "Model_dim (%s) must be even value, while this Model_dim mod 2 > 0." % model_dim
        if group is None and dist.is_available() and dist.is_initialized():
            group = dist.group.WORLD
        if 'pad_samples' in kwargs:
            logging.warning("`pad_samples` option in Moe-layer has been deprecated; "
                            "`pad_samples=False` is always assumed.")
            kwargs.pop('pad_samples')
        for k in kwargs:
            raise Exception('Unrecognized argument provided to Tutel Moe-layer: %s' % k)

        self.group = group
        self.result_func = result_func
        self.skip_moe = (int(os.environ.get('SKIP_MOE', '0')) != 0)
        self.index = index

        experts = dict(experts)
        self.num_local_experts = experts.pop('count_per_node', 1)
        self.num_global_experts = MOELayer.global_expert_count(self.num_local_experts, group)
        self.world_size = C.get_world_size(group)

        if self.num_global_experts < self.world_size:
            self.sharded_count = self.world_size // self.num_global_experts
            self.num_local_experts = 1
            self.ffn_zero_group = C.create_groups_from_world(
                group_count=self.num_global_experts).model_group
            self.shard_rank = C.get_world_rank(group) % self.sharded_count
        else:
            self.sharded_count, self.ffn_zero_group, self.shard_rank = 1, None, 0

        if self.sharded_count == 1:
            self.auto_parallel, self.use_model_parallel = False, False
        elif parallel_type == 'auto':
            self.auto_parallel, self.use_model_parallel = True, False
        else:
            self.auto_parallel, self.use_model_parallel = False, (parallel_type == 'model')

        self.model_dim = model_dim
        self.is_postscore = is_postscore
        self.batch_prioritized_routing = (batch_prioritized_routing or
                                          int(os.environ.get('BATCH_PRIO', 0)) != 0)
        self.normalize_gate = normalize_gate
        self.is_gshard_loss = is_gshard_loss
        self.a2a_ffn_overlap_degree = a2a_ffn_overlap_degree
        self.use_2dh = use_2dh
        self.compress_name = compress_name
        self.comm_name = comm_name

        if seeds is not None and seeds[1] is not None:
            torch.manual_seed(seeds[1])

        experts_type = experts.pop('type')
        if experts_type == 'custom':
            self.experts = experts['module']
        else:
            mod = _import_builtin('expert', experts_type)
            if experts_type == 'ffn':
                assert 'fused_custom_fn' not in experts, \
                    "`fused_custom_fn` option for Moe-layer has been deprecated."
                assert 'implicit_dropout_p' not in experts, \
                    "`implicit_dropout_p` option for Moe-layer has been deprecated."
            self.experts = mod.ExpertModule(**experts)
        self.experts_type = experts_type
        self.experts.update(self)

        for n, p in self.experts.named_parameters():
            if scan_expert_func is not None:
                scan_expert_func(n, p)
            setattr(p, '_tutel_expert', True)

        if isinstance(gate_type, str):
            assert re.match(r'^Top[0-9]+Gate$', gate_type), "Unrecognized gate_type: %s" % gate_type
            top_k = int(gate_type[3:-4])
            logging.warning("gate_type value `%s` has been deprecated, please use gate_type = "
                            "{'type': 'top', 'k': %d} instead." % (gate_type, top_k))
            gate_type = {'type': 'top', 'k': top_k}
        if not isinstance(gate_type, list):
            gate_type = [gate_type]

        gates = []
        for gi, spec in enumerate(gate_type):
            spec = dict(spec)
            kind = spec.pop('type')
            if seeds is not None and seeds[0] is not None:
                torch.manual_seed(seeds[0] + gi)
            try:
                mod = _import_builtin('gate', kind)
            except Exception:
                raise Exception("Unrecognized gate_type: %s" % kind)
            gate = mod.Gate(model_dim=self.model_dim, num_global_experts=self.num_global_experts,
                            **spec)
            if not hasattr(gate, 'gate_noise'):
                gate.gate_noise = spec.get('gate_noise', 0.0)
            if not hasattr(gate, 'capacity_factor'):
                gate.capacity_factor = spec.get(
                    'capacity_factor', float(os.environ.get('CAP_FACTOR', 1.0)))
            gate.gate_kind = kind
            gates.append(gate)
        self.gates = ModuleList(gates)

        if seeds is not None and len(seeds) > 2 and seeds[2] is not None:
            torch.manual_seed(seeds[2])
        self.save_count = 0
        self._scheduler = None
        self._fused = None
        self.last_stats = None
        from ..utils import metrics
        self.collect_stats = metrics.enabled_by_env()    # routing counters in last_stats (utils/metrics.py)

    # ------------------------------------------------------------------------------------
    def extra_repr(self):
        return 'Top-K(s) = %s, Total-Experts = %d [managed by %d device(s)],' % (
            ['k=%d, noise=%s' % (g.top_k, g.gate_noise) for g in self.gates],
            self.num_global_experts, self.world_size)

    def get_parameter_iterator(self, param_type):
        if param_type == 'gate':
            return self.gates.named_parameters()
        if param_type == 'local_experts':
            return self.experts.named_parameters()
        raise Exception("Specified parameter type is not recognized: %s. Valid `param_type` "
                        "includes: gate, local_experts." % param_type)

    def expert_local(self, x, reserve_shape):
        y = self.experts(x.view(x.size(0), x.size(1), *reserve_shape), self)
        self.protected_shape = y.shape
        return y.reshape(y.size(0), y.size(1), -1)

    # ------------------------------------------------------------------------------------
    def _plan(self, degree, x, gctx, top_k, cf, reserve_shape):
        """(degree, comm_name) of this call.  An integer degree and a named algorithm are used as given; 'auto'
        (degree 0 / 'auto', comm_name 'auto') goes through the adaptive scheduler, which calibrates at the first
        call, collectively over the layer's group, and then always returns the frozen plan."""
        degree_auto = isinstance(degree, str) or not degree
        comm_auto = self.comm_name == 'auto'
        if not degree_auto and not comm_auto:
            return int(degree), self.comm_name
        from ..parallel import scheduler
        if self._scheduler is None:
            self._scheduler = scheduler.AdaptiveScheduler.for_layer(self, x, top_k, cf, degree_auto=degree_auto)
            if not degree_auto:
                self._scheduler.degrees = [int(degree)]
        sched = self._scheduler
        if sched.frozen is None:
            E = self.num_global_experts
            base_cap = top_k * int(cf * ((x.size(0) + E - 1) // E)) if cf > 0 else 0

            def allowed(d):
                # chunks must divide the capacity once it is aligned to 4 * shards * d
                return d <= 32 and (base_cap == 0 or base_cap >= 4 * self.sharded_count * d)

            params = [p for p in self.parameters() if p.requires_grad]

            def run_candidate(d, comm):
                with torch.enable_grad():
                    xin = x.detach().requires_grad_(True)
                    y, l_aux = self._forward_core(xin, gctx, top_k, cf, int(d), reserve_shape,
                                                  comm_name=comm or self.comm_name)
                    outs = [y] if l_aux is None or not l_aux.requires_grad else [y, l_aux]
                    grads = [torch.ones_like(o) for o in outs]
                    torch.autograd.grad(outs, [xin] + params, grads, allow_unused=True)

            was_training = self.save_count
            sched.resolve(run_candidate, x.device, allowed_degree=allowed,
                          stage_split=lambda: self._roofline_stage_split(x, top_k, cf),
                          codec_info=self._codec_verdict(x, top_k, cf))
            self.save_count = was_training
        comm = sched.frozen_comm or (self.comm_name if not comm_auto else 'naive')
        return sched.frozen, comm

    def _roofline_stage_split(self, x, top_k, cf):
        """(send, ffn, return) times of one forward + backward at degree 1, from shapes: NVLink bytes at the
        measured peer bandwidth and expert FLOPs at the measured sustained bf16 rate.  Input of the scheduler's
        flow-shop model."""
        W, E = self.world_size, self.num_global_experts
        M = x.size(-1)
        H = getattr(self.experts, 'hidden_size_per_expert', M) // max(self.sharded_count, 1)
        C = top_k * int(max(cf, 1.0) * ((x.size(0) + E - 1) // E))
        wire = E * C * M * x.element_size() * (W - 1) / max(W, 1)
        if self.compress_name in ('int8', 'zfp'):
            wire /= 2.0
        t_link = 2.0 * wire / 770e9                              # forward + backward use each direction twice
        # per rank E_l * W * C rows through two GEMMs of 2 * M * H FLOPs per row, forward + dgrad + wgrad
        flops = 3.0 * 2.0 * 2.0 * max(E // max(W, 1), 1) * W * C * M * H
        t_ffn = flops / 1.4e15
        return t_link * 1e3, t_ffn * 1e3, t_link * 1e3

    def _codec_verdict(self, x, top_k, cf):
        """For a configured codec: whether, by the model, its encode + decode time is paid back by the bytes it
        takes off NVLink (kernels at their measured rates; recorded in the scheduler's report)."""
        if self.compress_name in ('no', None):
            return None
        from ..parallel import scheduler
        W, E = self.world_size, self.num_global_experts
        C = top_k * int(max(cf, 1.0) * ((x.size(0) + E - 1) // E))
        raw = E * C * x.size(-1) * x.element_size()
        rates = {'int8': (1800e9, 2300e9, 2.0), 'zfp': (190e9, 160e9, 2.0), 'lz': (20e9, 230e9, 1.2)}
        enc, dec, ratio = rates.get(self.compress_name, (1e12, 1e12, 1.0))
        t_raw = raw * (W - 1) / max(W, 1) / 770e9
        pays = scheduler.codec_pays_off(raw / enc, raw / dec, t_raw, ratio)
        return {'name': self.compress_name, 'ratio': ratio, 'pays_off_on_nvlink': bool(pays)}

    def _route(self, x, gctx, top_k, capacity_factor, degree):
        logits = gctx(x)
        if self.training and gctx.gate_noise > 0:
            noisy = logits + gctx.gate_noise * torch.randn_like(logits) / self.num_global_experts
        else:
            noisy = logits
        scores = F.softmax(noisy, dim=1)
        if self.is_gshard_loss:
            loss_fn = losses.gshard_loss
        else:
            def loss_fn(gates, topk_ids):
                return losses.load_importance_loss(
                    F.softmax(logits, dim=1), noisy.gather(index=topk_ids, dim=1),
                    self.num_global_experts, gctx.gate_noise)
        crit, l_aux = extract_critical(
            scores, top_k=top_k, loss_fn=loss_fn, capacity_factor=capacity_factor,
            batch_prioritized_routing=self.batch_prioritized_routing,
            normalize_gate=self.normalize_gate, group=self.group,
            alignment=4 * self.sharded_count * degree)
        return logits.dtype, crit, l_aux

    def _fused_path_ok(self, x, gctx, top_k, cf, degree, comm_name):
        """Whether this call can run on the fused sm_100a kernels; everything else takes the generic path."""
        if not x.is_cuda or os.environ.get('PLANMOE_FUSED', '1') == '0':
            return False
        if self.experts_type != 'ffn' or self.sharded_count != 1:
            return False
        if getattr(self.experts, 'skip_expert', False):
            return False
        # codecs: raw bf16 rows or int8 rows (quantised by the sender, de-quantised in front of the GEMM);
        # zfp / lz take the generic compress -> all-to-all -> decompress pipeline
        if self.compress_name not in fused_codecs():
            return False
        if self.compress_name == 'int8':
            # int8 rows: quantised per token before the send (so no gate scaling on the way: post-score layers),
            # 128-column groups in the push epilogue, the fused send as the carrier
            from ..ops import fused_moe as _fm
            out_dim = self.experts.batched_fc2_w.size(2)
            if not self.is_postscore or x.size(-1) % 128 or out_dim % 128 or not _fm._fuse_send(self.world_size) \
                    or (max(x.size(-1), out_dim) + 16) > _fm.MAX_ROW_BYTES:
                return False
        # on one NVSwitch domain the flat push is Pipe-A2A's equal (every peer is one hop away at full rate);
        # the hierarchical algorithms exist on the generic path
        if comm_name not in ('naive', 'pipe'):
            return False
        if getattr(gctx, 'gate_kind', None) not in ('top', 'cosine_top'):
            return False
        if self.num_global_experts > 64 or x.size(-1) % 64 != 0:
            return False
        from ..ops import fused_moe
        if min(int(top_k), self.num_global_experts) > fused_moe.MAX_TOP_K or int(degree) > fused_moe.MAX_CHUNKS:
            return False
        return self.experts.fused_ok(x)

    def forward(self, input, gate_index=0, capacity_factor=None, top_k=None,
                a2a_ffn_overlap_degree=None, reserve_dims=1):
        if self.skip_moe:
            out = input
            out.l_aux = None
            return self.result_func(out) if self.result_func is not None else out

        original_shape, original_dtype = input.shape, input.dtype
        assert len(original_shape) >= 2, \
            "Input data must be at least 2D tensor: (s)amples, .., (m)odel_dim"
        x = input.reshape(-1, original_shape[-reserve_dims:].numel())
        for p in self.experts.parameters():
            x = x.to(p.dtype)
            break
        gctx = self.gates[gate_index]
        degree = self.a2a_ffn_overlap_degree if a2a_ffn_overlap_degree is None \
            else a2a_ffn_overlap_degree
        top_k = gctx.top_k if top_k is None else top_k
        cf = gctx.capacity_factor if capacity_factor is None else capacity_factor
        reserve_shape = original_shape[-reserve_dims:]
        degree, comm_name = self._plan(degree, x, gctx, top_k, cf, reserve_shape)
        if self.training:
            self.save_count += 1
        y, l_aux = self._forward_core(x, gctx, top_k, cf, int(degree), reserve_shape, comm_name)

        y = y.view(list(original_shape)).to(original_dtype)
        self.l_aux = y.l_aux = l_aux
        return self.result_func(y) if self.result_func is not None else y

    def _forward_core(self, x, gctx, top_k, cf, degree, reserve_shape, comm_name=None):
        comm_name = comm_name or self.comm_name
        if self._fused_path_ok(x, gctx, top_k, cf, degree, comm_name):
            from ..ops import fused_moe
            return fused_moe.forward(self, x, gctx, top_k, cf, int(degree))
        return self._generic_forward(x, gctx, top_k, cf, int(degree), reserve_shape, comm_name)

    def _generic_forward(self, x, gctx, top_k, cf, degree, reserve_shape, comm_name=None):
        comm_name = comm_name or self.comm_name
        if x.is_cuda:
            with torch.autocast('cuda', enabled=False):
                logits_dtype, crit, l_aux = self._route(x, gctx, top_k, cf, degree)
        else:
            logits_dtype, crit, l_aux = self._route(x, gctx, top_k, cf, degree)

        y = fast_encode(x.to(logits_dtype), crit, self.is_postscore).to(x.dtype)   # [E, C, M]

        if self.auto_parallel:
            self.use_model_parallel = (
                y.numel() * (self.sharded_count - 1) * 2 <
                sum(p.numel() for p in self.experts.parameters()))
        if self.num_global_experts < self.world_size:
            if self.use_model_parallel:
                y = y.repeat(1, self.sharded_count, 1).view(self.world_size, -1, y.size(2))
            else:
                y = y.view(self.world_size, -1, y.size(2))

        def expert_fn(expert_input):
            return self.expert_local(expert_input, reserve_shape)

        y = a2a_ffn_overlap_forward(
            y, expert_fn=expert_fn, a2a_ffn_overlap_degree=degree, use_2dh=self.use_2dh,
            group=self.group, compress_name=self.compress_name, comm_name=comm_name)

        if self.num_global_experts < self.world_size:
            if self.use_model_parallel:
                y = y.view(self.num_global_experts, self.sharded_count, -1, y.size(2)).sum(dim=1)
            else:
                y = y.view(self.num_global_experts, -1, y.size(2))

        y = fast_decode(y.to(logits_dtype), crit, self.is_postscore)
        self.last_stats = dict(capacity=int(crit[4]), degree=degree, path='generic', comm=comm_name)
        if self.collect_stats:
            from ..utils import metrics
            self.last_stats.update(metrics.routing_stats(crit[1], crit[2], self.num_global_experts, int(crit[4])))
            self.last_stats.update(metrics.wire_stats(self.num_global_experts, int(crit[4]), x.size(-1),
                                                      x.element_size(), self.world_size, self.compress_name,
                                                      comm_name, degree))
        return y, l_aux


moe_layer = MOELayer
