"""MoBA-style routing as a second producer of block lists for the selected branch.
Same entry points as the reference's nsa/triton/moba.py (`_per_query_top_k_indices` :18-92,
`moba_attention` :95-125): per-query-token top-k block routing, aggregated per query block, then the
selected-attention kernel over the listed blocks."""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

from . import _lib as L
from . import ops
from .selected import selected_attention


def _per_query_top_k_indices(Q: torch.Tensor, K: torch.Tensor, *, block_size_n: int, block_size_m: int, top_k_per_query: int,
                             top_k_cap: int, causal: bool, scale: float) -> torch.Tensor:
    """int32 [B,H,nq,cap], cap = min(top_k_cap, nk): the union of the query block's rows' picks in ascending order,
    padded with the out-of-range id nk (which the selected kernel skips); a union larger than the cap keeps the cap
    blocks with the best block-level score, best first.  Ties go to the lowest block id; rows with fewer legal
    blocks than picks contribute their legal ones only (the reference's torch.topk returns arbitrary illegal ids
    there, which its attention kernel skips -- the attended set is the same)."""
    ops._need_cuda(Q, K)
    assert Q.dtype in (torch.float16, torch.bfloat16) and K.dtype == Q.dtype
    B, H, Tq, D = Q.shape
    Hkv, Tk = K.shape[1], K.shape[2]
    bm, bn = int(block_size_m), int(block_size_n)
    nq, nk = (Tq + bm - 1) // bm, (Tk + bn - 1) // bn
    cap = min(int(top_k_cap), nk)
    kq = min(int(top_k_per_query), nk)
    Qc = ops._dense(Q, "Q")
    Kb = ops.pool_mean(K, bn)
    idx = torch.empty((B, H, nq, cap), device=Q.device, dtype=torch.int32)
    with torch.cuda.device(Q.device):
        L.check(L.load().nsa_moba_block_indices(Qc.data_ptr(), Kb.data_ptr(), idx.data_ptr(), B, H, Hkv, Tq, nq, nk, D, kq, cap, bm, bn,
                                                nk * bn - nq * bm, int(bool(causal)), float(scale), L.dtype_code(Q.dtype),
                                                L.stream_ptr()), "nsa_moba_block_indices")
    return idx


def moba_attention(Q: torch.Tensor, K: torch.Tensor, V: torch.Tensor, *, block_size_n: int = 64, block_size_m: int = 64,
                   top_k_per_query: int = 16, top_k_cap: int = 64, causal: bool = True,
                   scale: Optional[float] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-query top-k block routing, then attention over the union-gathered blocks (out, lse)."""
    D = Q.shape[-1]
    s = float(scale) if scale is not None else 1.0 / math.sqrt(D)
    idx = _per_query_top_k_indices(Q, K, block_size_n=block_size_n, block_size_m=block_size_m, top_k_per_query=top_k_per_query,
                                   top_k_cap=top_k_cap, causal=causal, scale=s)
    return selected_attention(Q, K, V, block_size_n=block_size_n, block_size_m=block_size_m, top_k=idx.shape[-1],
                              block_indices=idx, causal=causal, scale=scale)


__all__ = ["moba_attention"]
