"""Selected branch: each query block attends the KV blocks listed for it.
Same signature as the reference's nsa/triton/selected.py:188-201."""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib as L
from . import ops


def _topk_indices_from_scores(block_scores, top_k, n_q_blocks, n_kv_blocks, block_size_m, block_size_n, Tq, Tk,
                              causal, device=None) -> torch.Tensor:
    """int32 [B,H,nq,k] from caller scores; legality uses the unpadded offset Tk-Tq
    (nsa/triton/selected.py:153-185).  Ties go to the lowest block index."""
    assert block_scores.shape[-2:] == (n_q_blocks, n_kv_blocks)
    return ops.topk_from_scores(block_scores, top_k=top_k, bm=block_size_m, bn=block_size_n, offset=Tk - Tq,
                                causal=bool(causal))


def selected_attention(
    Q: torch.Tensor, K: torch.Tensor, V: torch.Tensor, block_size_n: int = 64, block_size_m: int = 64,
    top_k: int = 16, block_scores: Optional[torch.Tensor] = None, block_indices: Optional[torch.Tensor] = None,
    causal: bool = True, scale: Optional[float] = None, num_warps: int = 4, num_stages: int = 2,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Returns (out [B,H,Tq,D], lse fp32 [B,H,Tq]); lse is -inf (and out 0) for rows whose
    listed blocks hold no visible key.  `block_indices` [B,H|Hkv,nq,k] wins over
    `block_scores` [B,H,nq,nk]; one of them is required.  Lengths need not be multiples of
    the block sizes (the kernel treats the missing tail as zero keys, like the reference's
    padding).  Ids outside [0,nk) are skipped.  num_warps/num_stages are accepted and ignored."""
    assert Q.dtype in (torch.float16, torch.bfloat16), "Q must be fp16 or bf16"
    assert K.dtype == Q.dtype and V.dtype == Q.dtype
    assert Q.is_cuda and K.is_cuda and V.is_cuda
    B, H, Tq, D = Q.shape
    Hk, Tk = K.shape[1], K.shape[2]
    assert K.shape == V.shape == (B, Hk, Tk, D) and H % Hk == 0
    n_q_blocks = (Tq + block_size_m - 1) // block_size_m
    n_kv_blocks = (Tk + block_size_n - 1) // block_size_n
    if block_indices is None:
        assert block_scores is not None, "selected_attention requires either block_scores or block_indices"
        assert block_scores.shape == (B, H, n_q_blocks, n_kv_blocks), (
            f"block_scores shape {tuple(block_scores.shape)} != {(B, H, n_q_blocks, n_kv_blocks)}")
        block_indices = _topk_indices_from_scores(block_scores.float(), top_k, n_q_blocks, n_kv_blocks, block_size_m,
                                                  block_size_n, Tq, Tk, causal, Q.device)
    else:
        assert block_indices.shape[0] == B and block_indices.shape[1] in (H, Hk) and block_indices.shape[2] == n_q_blocks
    out, lse = ops.attention_fwd(
        Q, K, V, branches=L.BRANCH_SELECTED, fused=False, causal=bool(causal), scale=ops.softmax_scale(D, scale),
        idx=block_indices, bm=block_size_m, bn=block_size_n)
    return out, lse


__all__ = ["selected_attention"]
