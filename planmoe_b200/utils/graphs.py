"""CUDA-graph capture of whole training steps.

A step of the fused MoE layer is a few dozen short kernels, so an eager loop is bound by Python and
launch overhead rather than by the GPU.  ``GraphedSteps`` captures ``unroll`` consecutive calls of a
step function (forward + backward + optimizer) into one CUDA graph and replays it.

What makes the layer capturable: every kernel argument is either a shape or an address that stays
fixed between replays (buffers come from the graph's private pool or from the symmetric heap), and
the expected flag counts of the peer-to-peer protocol live in device memory and are advanced by
kernels inside the graph (``ops/fused_moe.py``).  ``unroll`` must be a multiple of 2 for the fused
layer: it alternates between two sets of receive buffers from step to step, and a graph has to
contain the whole cycle.  With several ranks every rank replays the same graph the same number of
times; the kernels inside still wait for their peers' flags.

Rules for the step function: no host synchronisation, no collective of the control plane, static
input tensors (copy new data into them between replays), adaptive pipeline degree already frozen.
Before capturing a model that has already run backward on the default stream, drop every reference
to its last autograd graph (``layer.l_aux = None``, old losses): gradient accumulators that stay
alive keep the default stream, and work on the default stream invalidates a capture.

If capture fails, the constructor restores the current stream and the allocator before re-raising,
so the caller can continue eagerly.
"""

import gc

import torch


class GraphedSteps:
    def __init__(self, step_fn, unroll=2, warmup=3, split=False):
        """``step_fn()`` runs one step on static inputs and returns a tensor (the loss) or None.

        ``split=True`` captures every one of the ``unroll`` steps as a graph of its own (one shared memory pool;
        replay them in capture order, cyclically): ``replay_one(i)`` then runs a single step, so a caller that
        feeds each step its own input can overlap the copy for step i + 1 with step i."""
        assert unroll >= 1
        self.unroll = unroll
        self.split = bool(split)
        self.outputs = []
        self.graphs = []
        gc.collect()
        prev = torch.cuda.current_stream()
        side = torch.cuda.Stream()
        side.wait_stream(prev)
        with torch.cuda.stream(side):                      # warm up on the stream the capture will use
            for _ in range(max(warmup, 2) * unroll):
                step_fn()
        prev.wait_stream(side)
        torch.cuda.synchronize()
        n_graphs = unroll if self.split else 1
        per_graph = 1 if self.split else unroll
        for gi in range(n_graphs):
            graph = torch.cuda.CUDAGraph()
            kw = {'pool': self.graphs[0].pool()} if self.graphs else {}
            ctx = torch.cuda.graph(graph, stream=side, **kw)
            began = False
            try:
                ctx.__enter__()
                began = True
                for _ in range(per_graph):
                    self.outputs.append(step_fn())
                ctx.__exit__(None, None, None)
            except BaseException:
                # torch.cuda.graph does not unwind when ending the capture fails: do it here
                if began:
                    try:
                        graph.capture_end()
                    except Exception:
                        pass
                    try:
                        torch._C._cuda_endAllocateToPool(torch.cuda.current_device(), graph.pool())
                    except Exception:
                        pass
                torch.cuda.set_stream(prev)
                try:
                    torch.cuda.synchronize()
                except Exception:
                    pass
                self.outputs = []
                self.graphs = []
                raise
            self.graphs.append(graph)
        self.graph = self.graphs[0]

    def replay(self):
        """Run ``unroll`` steps; returns the list of per-step outputs (static tensors, overwritten by the
        next replay)."""
        for g in self.graphs:
            g.replay()
        return self.outputs

    def replay_one(self, i):
        """Split mode: run step ``i`` of the cycle (call with i = 0, 1, ..., unroll - 1, 0, ... in that order)."""
        assert self.split, "replay_one needs split=True"
        self.graphs[i].replay()
        return self.outputs[i]
