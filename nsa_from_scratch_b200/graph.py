"""The forward step as one CUDA graph.

At short sequences the six launches of a forward (two block-mean pools, score + top-k, two K/V pools, the
fused attention kernel) and the host code between them cost more than the kernels run; captured once and
replayed, the step is a single graph launch.  The graph reads and writes the tensors it was captured on:
refill them in place (`Q.copy_(...)`) and call the object again.
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import Tensor

from .forward import nsa_forward


class GraphedForward:
    """`nsa_forward(Q, K, V, cfg, gate_logits=...)` captured on the given device tensors.  Calling the object
    replays the graph on the current stream and returns the (static) output tensor."""

    def __init__(self, Q: Tensor, K: Tensor, V: Tensor, cfg, *, gate_logits: Optional[Tensor] = None, warmup: int = 2):
        if not (Q.is_cuda and K.is_cuda and V.is_cuda):
            raise ValueError("GraphedForward captures device tensors")
        self.Q, self.K, self.V, self.gate_logits, self.cfg = Q, K, V, gate_logits, cfg
        side = torch.cuda.Stream(Q.device)
        side.wait_stream(torch.cuda.current_stream(Q.device))
        with torch.cuda.stream(side), torch.no_grad():
            for _ in range(max(1, warmup)):          # first calls set kernel attributes and warm the allocator
                nsa_forward(Q, K, V, cfg, gate_logits=gate_logits)
        torch.cuda.current_stream(Q.device).wait_stream(side)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph), torch.no_grad():
            self.out = nsa_forward(Q, K, V, cfg, gate_logits=gate_logits)

    def __call__(self) -> Tensor:
        self.graph.replay()
        return self.out


__all__ = ["GraphedForward"]
