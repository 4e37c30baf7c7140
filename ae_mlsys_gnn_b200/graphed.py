"""One training step of fixed shapes as a CUDA graph.

The small benchmark configurations (a 2,708-node GAT, a 19,717-node MoNet, 32 point clouds)
run a few dozen kernels of 5-50 microseconds per epoch: launched one by one through Python
their epoch is host launch time, not kernel time.  Capturing forward, loss, backward and the
optimizer update once and replaying the graph removes the host from the loop.  Nothing in the
reference corresponds to this (its scripts launch eagerly, script/train/train_gatconv_our.py:184-200).

Requirements, all met by the operators of this package: no host synchronisation inside the
step (graph-static maps such as the CSR-to-CSC positions are built by the warm-up steps),
memory from torch's allocator (the graph's private pool keeps addresses fixed between
replays), an optimizer created with ``capturable=True``.  Inputs are read from the tensors
the step function closes over: copy new values into them before ``replay()``.
"""
from __future__ import annotations

import torch


class GraphedStep:
    def __init__(self, step_fn, warmup: int = 3, device=None):
        """``step_fn()`` runs one whole step and returns a tensor (e.g. the loss), which the
        replays keep updating in place."""
        dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.device = dev
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for _ in range(max(1, warmup)):
                step_fn()
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.result = step_fn()

    def replay(self):
        self.graph.replay()
        return self.result

    __call__ = replay
