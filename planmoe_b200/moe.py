"""Facade: the MoE layer and the routing / dispatch helpers (reference ``PlanMoE/moe.py:6-12``)."""

from .jit_kernels.gating import fast_cumsum_sub_one
from .impls.fast_dispatch import fast_dispatcher, extract_critical, fast_encode, fast_decode

top_k_routing = extract_critical

from .impls.moe_layer import moe_layer  # noqa: E402
