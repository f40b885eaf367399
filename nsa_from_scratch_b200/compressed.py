"""Compressed branch: mean-pool K/V, attend over the pooled tokens.
Same signature as the reference's nsa/triton/compressed.py:191-199 (+ keyword `stride_c`)."""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib as L
from . import ops


def _mean_pool(x: torch.Tensor, block_c: int) -> torch.Tensor:
    """[B,H,T,D] -> [B,H,ceil(T/block_c),D]; trailing partial block divided by block_c
    (nsa/triton/compressed.py:25-44)."""
    return ops.pool_mean(x, block_c)


def compressed_attention(
    Q: torch.Tensor, K: torch.Tensor, V: torch.Tensor, block_size_c: int = 64, pool: str = "mean",
    causal: bool = True, scale: Optional[float] = None, *, stride_c: Optional[int] = None,
    pool_proj_k: Optional[torch.Tensor] = None, pool_proj_v: Optional[torch.Tensor] = None,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Returns (out [B,H,Tq,D] in Q's dtype, lse fp32 [B,H,Tq]).  Rows with no visible pooled
    token give out 0 / lse -inf.  K/V may carry fewer (grouped) heads than Q.
    pool="learned" (forward only): pooled token = sum_s K[c*stride+s] * pool_proj_k[s] with pool_proj_* [block_size_c, D],
    the reference's plain-torch rule (nsa/reference.py:109-113; its own kernel wrapper refuses it,
    nsa/triton/compressed.py:219-220)."""
    if pool not in ("mean", "learned"):
        raise ValueError(f"unknown pool: {pool}")
    if pool == "learned" and (pool_proj_k is None or pool_proj_v is None):
        raise ValueError("compressed_attention: pool='learned' needs pool_proj_k and pool_proj_v")
    assert Q.dtype in (torch.float16, torch.bfloat16), "Q must be fp16 or bf16"
    assert K.dtype == Q.dtype and V.dtype == Q.dtype
    assert Q.is_cuda and K.is_cuda and V.is_cuda
    assert Q.dim() == 4 and K.dim() == 4 and V.dim() == 4
    B, H, Tq, D = Q.shape
    Bk, Hk, Tk, Dk = K.shape
    assert (B, D) == (Bk, Dk) and H % Hk == 0, "Q and K must agree on B, D and head grouping"
    assert V.shape == K.shape
    assert D in (32, 64, 128), f"unsupported head dim D={D}"
    stride = block_size_c if stride_c is None else int(stride_c)
    if pool == "learned":
        Kc = ops.pool_learned(K, pool_proj_k, block_size_c, stride)
        Vc = ops.pool_learned(V, pool_proj_v, block_size_c, stride)
    else:
        Kc = ops.pool_mean(K, block_size_c, stride)
        Vc = ops.pool_mean(V, block_size_c, stride)
    Tk_pad = Kc.shape[2] * block_size_c if stride == block_size_c else Tk
    out, lse = ops.attention_fwd(
        Q, K, V, branches=L.BRANCH_COMPRESSED, fused=False, causal=bool(causal),
        scale=ops.softmax_scale(D, scale), Kc=Kc, Vc=Vc, cmp_block=block_size_c, cmp_stride=stride,
        cmp_offset=Tk_pad - Tq)
    return out, lse


__all__ = ["compressed_attention"]
