// Symmetric heap, status word and raw-pointer tensor views.
//
// The data plane of the MoE layer is SM-driven stores into peer GPUs' memory.  Each rank
// allocates one device region ("heap"), exports it as a CUDA IPC handle, and maps every peer's
// region; the table of peer base addresses lives in device memory so kernels can turn
// (rank, byte offset) into an address.  Allocation inside the heap is a bump allocator driven
// from Python in the same order on every rank, so offsets agree without communication.
//
// This replaces the reference's private NCCL communicator set
// (PlanMoE/custom/custom_kernel.cpp:130-176): no ncclSend/ncclRecv is issued on the data plane.
#pragma once

#include <pybind11/pybind11.h>

void bind_symm_heap(pybind11::module_& m);
