"""One typed view of the configuration surface.

The reference is configured through three uncoordinated mechanisms: constructor keywords of ``moe_layer``
(PlanMoE/impls/moe_layer.py:44-75), environment variables read all over the code, and string-keyed native
registries (PlanMoE/custom/custom_kernel.cpp:194-224).  All three are kept verbatim (keywords and variable names are
the public contract); this module adds what was missing: a single place that names every switch, says what it does,
and resolves keywords + environment into one object.

``MoEConfig.from_kwargs(**layer_kwargs)`` validates the keywords of a layer the way the layer itself does and returns a
dataclass; ``MoEConfig.from_layer(layer)`` reads one back from a built layer; ``runtime_env()`` returns the current
value of every environment switch; ``ENV`` is the documentation table (also printed by ``python -m
planmoe_b200.utils.config``).
"""

import dataclasses
import os
from typing import Any, Optional, Union

# name -> (default, meaning).  Reference switches first (names kept verbatim), then this package's own.
ENV = {
    # ---- switches of the reference ------------------------------------------------------------------------------
    'SKIP_MOE': ('0', 'moe_layer.forward returns its input unchanged (ablation timing)'),
    'SKIP_EXPERT': ('0', 'expert FFN returns its input unchanged; such layers take the generic path'),
    'SKIP_A2A': ('0', 'every all-to-all of the generic path is the identity'),
    'BATCH_PRIO': ('0', 'batch-prioritised routing for every layer (same as batch_prioritized_routing=True)'),
    'CAP_FACTOR': ('1.0', 'capacity factor of gates built without one'),
    'FAST_CUMSUM': ('1', '0: torch.cumsum instead of the scan kernel behind fast_cumsum_sub_one'),
    'LOCAL_SIZE': ('world size', 'ranks per logical group for pipe / dd / hetu (4 on one 8-GPU box = two groups)'),
    'LOCAL_RANK': ('0', 'rank within the node: CUDA device and NUMA binding'),
    'USE_NVRTC': ('1', 'jit.create_cuda_kernel: 0 compiles with an nvcc child process instead of NVRTC'),
    'TUTEL_CUDA_SANDBOX': ('0', 'launcher.execl: 2 pins CUDA_VISIBLE_DEVICES to LOCAL_RANK; also disables NUMA binding'),
    'NUMA_TYPE': ('1', 'system.init_affinity_at_program_beginning: local ranks per NUMA node (<= 0: no binding)'),
    'OMP_NUM_THREADS': ('set by the launchers', 'CPU threads per rank'),
    'MOE / L_AUX_WT / NO_OVERFLOW': ('0 / 0 / 0', 'fairseq integration: every n-th layer is MoE, weight of the auxiliary '
                                     'loss, zero non-finite gradients'),
    'STRICT_FMT / PTYPE / CONFIG / DEVICE / MODE / CONFIG_STORE_PATH / HOSTS / VERBOSE': ('', 'parted (auto-SPMD tool)'),
    # ---- this package --------------------------------------------------------------------------------------------
    'PLANMOE_FUSED': ('1', '0: every layer takes the generic path (ATen routing, codec objects, stand-alone all-to-all)'),
    'PLANMOE_FUSE_SEND': ('1', '0: the dispatch send is a separate copy kernel in front of the flag-gated GEMM instead of a '
                          'copy warp inside it (the int8 wire needs 1)'),
    'PLANMOE_GEMM': ('tcgen05', "'cublas': FFN experts use torch.matmul (and layers leave the fused path)"),
    'PLANMOE_GEMM_CTA_GROUP': ('auto', '1 or 2: force one-CTA (128 x 256) or two-CTA (256 x 256) tiles'),
    'PLANMOE_GEMM_TMA_STORE': ('1', '0: epilogues write with 16-byte stores instead of bulk tensor stores'),
    'PLANMOE_GEMM_COPY_VARIANT': ('0', '1: plain launches use the kernel variant that carries the dispatch send (one ring '
                                  'stage less); for measuring that variant alone'),
    'PLANMOE_LOCAL_FIRST': ('0', '0: the dispatch send interleaves all destinations from the first row and the tile loop '
                            'visits sources round-robin; 1: own rows are sent and consumed first (measured slower)'),
    'PLANMOE_GEMM_TRACE': ('0', '1: fused launches record per-CTA role timestamps; fused_moe.last_trace() summarises them'),
    'PLANMOE_COPY_DBG': ('0', 'bit 0: fence + release on every flag add of the dispatch send; bit 1: all flag adds at the end '
                         '(experiments)'),
    'PLANMOE_WAIT_BUDGET_MS': ('20000', 'how long a device-side wait (flag or mbarrier) may last before the kernel records an '
                               'error and returns'),
    'PLANMOE_HEAP_MB': ('1024', 'size of a symmetric-heap segment'),
    'PLANMOE_DEBUG_GUARDS': ('0', '1: canary bands around heap blocks (checked by Transport.check) and NaN-filled receive '
                             'buffers; host-side range and ownership assertions on the routing tensors'),
    'PLANMOE_PLAN_CACHE': ('~/.cache/planmoe_b200/plans.json', 'where the adaptive scheduler stores frozen plans'),
    'PLANMOE_PLAN_CACHE_DISABLE': ('0', '1: always calibrate'),
    'PLANMOE_STAGE_TIMERS': ('0', '1: CUDA events + NVTX ranges around every stage of the fused layer'),
    'PLANMOE_STATS': ('0', '1: layer.last_stats carries routed / dropped token counts and wire bytes'),
    'PLANMOE_NO_NATIVE': ('0', '1: CPU paths avoid the native extension'),
}


def runtime_env():
    """{switch: current value or None} for every single-name switch of ``ENV``."""
    return {k: os.environ.get(k) for k in ENV if ' ' not in k}


@dataclasses.dataclass
class MoEConfig:
    """Everything that configures one ``moe_layer`` (constructor keywords of the reference, same names and defaults)."""
    gate_type: Any = None                      # dict, list of dicts, or legacy 'Top<k>Gate'
    model_dim: int = 0
    experts: Optional[dict] = None             # {'type': 'ffn'|'custom', 'count_per_node', 'hidden_size_per_expert', ...}
    a2a_ffn_overlap_degree: Union[int, str] = 1    # int, or 'auto' / 0 for the adaptive scheduler
    is_postscore: bool = True
    batch_prioritized_routing: bool = False
    normalize_gate: bool = True
    is_gshard_loss: bool = True
    parallel_type: str = 'auto'                # 'auto' | 'data' | 'model' (sharded experts)
    use_2dh: bool = False
    index: int = 0
    compress_name: str = 'no'                  # 'no' | 'int8' | 'zfp' | 'lz' | a registered codec
    comm_name: str = 'naive'                   # 'naive' | 'pipe' | 'dd' | 'hetu' | 'nccl' | 'auto' | a registered comm
    seeds: Optional[tuple] = None

    _KEYS = ('gate_type', 'model_dim', 'experts', 'a2a_ffn_overlap_degree', 'is_postscore', 'batch_prioritized_routing',
             'normalize_gate', 'is_gshard_loss', 'parallel_type', 'use_2dh', 'index', 'compress_name', 'comm_name', 'seeds')

    @classmethod
    def from_kwargs(cls, **kw):
        kw = dict(kw)
        kw.pop('pad_samples', None)                                  # deprecated and ignored, as in the reference
        extra = {k: kw.pop(k) for k in ('scan_expert_func', 'result_func', 'group') if k in kw}
        for k in kw:
            if k not in cls._KEYS:
                raise Exception('Unrecognized argument provided to Tutel Moe-layer: %s' % k)
        cfg = cls(**kw)
        cfg.validate()
        cfg.callbacks = extra
        return cfg

    @classmethod
    def from_layer(cls, layer):
        return cls(gate_type=[{'type': getattr(g, 'gate_kind', 'top'), 'k': g.top_k, 'capacity_factor': g.capacity_factor,
                               'gate_noise': g.gate_noise} for g in layer.gates],
                   model_dim=layer.model_dim,
                   experts={'type': layer.experts_type, 'count_per_node': layer.num_local_experts,
                            'hidden_size_per_expert': getattr(layer.experts, 'hidden_size_per_expert', None)},
                   a2a_ffn_overlap_degree=layer.a2a_ffn_overlap_degree, is_postscore=layer.is_postscore,
                   batch_prioritized_routing=layer.batch_prioritized_routing, normalize_gate=layer.normalize_gate,
                   is_gshard_loss=layer.is_gshard_loss, use_2dh=layer.use_2dh, index=layer.index,
                   compress_name=layer.compress_name, comm_name=layer.comm_name)

    def validate(self):
        assert self.model_dim % 2 == 0, "Model_dim (%s) must be even value, while this Model_dim mod 2 > 0." % self.model_dim
        d = self.a2a_ffn_overlap_degree
        assert d in ('auto', 0) or (isinstance(d, int) and 1 <= d <= 32), \
            "a2a_ffn_overlap_degree must be an int in [1, 32], or 'auto' / 0"
        assert self.parallel_type in ('auto', 'data', 'model'), "parallel_type must be auto, data or model"
        return self

    def layer_kwargs(self):
        """Keywords to construct the layer this object describes."""
        out = {k: getattr(self, k) for k in self._KEYS}
        out.update(getattr(self, 'callbacks', {}))
        return out

    def build(self):
        from ..impls.moe_layer import MOELayer
        return MOELayer(**self.layer_kwargs())


def main():
    width = max(len(k) for k in ENV)
    for k, (default, meaning) in ENV.items():
        print('%-*s  default %-12s  %s' % (width, k, default, meaning))


if __name__ == '__main__':
    main()
