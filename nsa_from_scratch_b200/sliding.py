"""Sliding-window branch.  Same signature as the reference's nsa/triton/sliding.py:136-143."""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib as L
from . import ops


def sliding_attention(Q: torch.Tensor, K: torch.Tensor, V: torch.Tensor, window_size: int = 512, causal: bool = True,
                      scale: Optional[float] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Causal: keys [p-W+1, p]; symmetric: |j-p| <= W, with p = i + (Tk-Tq).
    Returns (out, lse fp32 [B,H,Tq])."""
    assert Q.is_cuda and K.is_cuda and V.is_cuda, "sliding_attention requires CUDA tensors"
    assert Q.dtype in (torch.float16, torch.bfloat16), "Q dtype must be fp16 or bf16"
    assert K.dtype == Q.dtype and V.dtype == Q.dtype, "K, V dtype must match Q"
    assert Q.shape[-1] == K.shape[-1] == V.shape[-1], "head dims must match"
    assert K.shape[0] == Q.shape[0] and Q.shape[1] % K.shape[1] == 0 and V.shape == K.shape
    assert window_size >= 1, "window_size must be >= 1"
    D = Q.shape[-1]
    assert D in (32, 64, 128), f"unsupported head dim D={D}"
    return ops.attention_fwd(Q, K, V, branches=L.BRANCH_SLIDING, fused=False, causal=bool(causal),
                             scale=ops.softmax_scale(D, scale), window=int(window_size))


__all__ = ["sliding_attention"]
