"""Facade: run-time compiled user kernels (reference ``PlanMoE/jit.py:4``)."""

from .impls.jit_compiler import create_cuda_kernel  # noqa: F401
