// Run-time compilation of user CUDA kernels with NVRTC for sm_100a.
//
// Counterpart of the reference's JIT engine (PlanMoE/custom/jit.h:62-324: nvcc / NVRTC ->
// cuModuleLoadDataEx -> cuLaunchKernel).  Differences: the target is always sm_100a, NVRTC and
// the driver entry points are resolved lazily (the extension imports on machines without a
// GPU), and kernels launch on the caller's stream instead of the default stream.
#pragma once

#include <pybind11/pybind11.h>

void bind_jit(pybind11::module_& m);
