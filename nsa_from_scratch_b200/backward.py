"""Selected-branch backward.  Same signature as the reference's nsa/triton/backward.py:125-140
(+ keyword `return_fp32`)."""
from __future__ import annotations

import torch

from . import ops


def selected_backward(
    dO: torch.Tensor, Q: torch.Tensor, K: torch.Tensor, V: torch.Tensor, O: torch.Tensor, LSE: torch.Tensor,
    block_indices: torch.Tensor, *, block_size_m: int, block_size_n: int, causal: bool, scale: float, Tq: int,
    Tk: int, return_fp32: bool = False,
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Inputs are the PADDED tensors the forward saw (lengths multiples of the block sizes);
    the causal offset is Tk_p - Tq_p as in the reference (backward.py:185).  Returns padded
    (dQ, dK, dV) in the input dtype, or in fp32 when return_fp32.  With grouped KV heads dK/dV
    are [B,Hkv,Tk_p,D], summed over the query heads of each group."""
    assert Q.dtype in (torch.float16, torch.bfloat16), "selected_backward: Q must be fp16/bf16"
    assert K.dtype == Q.dtype and V.dtype == Q.dtype and O.dtype == Q.dtype and dO.dtype == Q.dtype
    assert LSE.dtype == torch.float32
    assert block_indices.dtype == torch.int32
    Tq_p, Tk_p = Q.shape[2], K.shape[2]
    delta = ops.bwd_delta(dO, O)
    dQ, dK, dV = ops.selected_bwd(dO, Q, K, V, LSE, delta, block_indices, bm=block_size_m, bn=block_size_n,
                                  causal=bool(causal), scale=float(scale), offset=Tk_p - Tq_p, dq_fp32=return_fp32)
    if return_fp32:
        return dQ, dK, dV
    return dQ, ops.cast_from_f32(dK, K.dtype), ops.cast_from_f32(dV, V.dtype)


__all__ = ["selected_backward"]
