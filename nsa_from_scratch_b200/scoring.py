"""Selection scored from the compressed branch's attention probabilities (the NSA paper's scorer).

The reference scores selection blocks with block means (nsa/triton/forward.py:321-359); its functions take
scores or indices from outside through `block_scores=` / `block_indices=` (nsa/triton/selected.py:195-196),
which is how this scorer enters: `compressed_block_scores` gives fp32 scores of the reference's
`block_scores` shape, `select_blocks_compressed` the int32 indices.  `NSAConfig(scorer="compressed")` makes
`nsa_forward` use it.

score[query block, selection block] = sum over the block's 64 query rows (and, with one list per KV head,
over the heads that share it) of the compressed-attention probability mass that falls into the selection
block -- a compressed token's probability is split over the selection blocks its window overlaps, in
proportion to the overlap.
"""
from __future__ import annotations

from typing import Tuple

import torch
from torch import Tensor

from . import _lib as L
from . import ops


def _geometry(cfg, Tq: int, Tk: int) -> Tuple[int, int, int, int, int]:
    bc = int(cfg.block_size_c)
    stride = bc if getattr(cfg, "stride_c", None) is None else int(cfg.stride_c)
    n_c = ops.n_pooled(Tk, bc, stride)
    cmp_offset = (n_c * bc if stride == bc else Tk) - Tq
    bm, bn = int(cfg.block_size_m), int(cfg.block_size_n)
    if bm != 64:
        raise NotImplementedError("compressed-probability scoring takes 64-row query blocks")
    nq, nk = (Tq + bm - 1) // bm, (Tk + bn - 1) // bn
    return bc, stride, cmp_offset, nk, nk * bn - nq * bm


def compressed_block_scores(Q: Tensor, K: Tensor, cfg) -> Tensor:
    """fp32 [B,H|Hkv,nq,nk]: -inf on causally illegal blocks, +inf on forced ones (cfg.force_first / force_local)."""
    B, H, Tq, D = Q.shape
    Tk = K.shape[2]
    scale = float(cfg.scale if cfg.scale is not None else 1.0 / (D ** 0.5))
    bc, stride, cmp_offset, nk, sel_offset = _geometry(cfg, Tq, Tk)
    Kc = ops.pool_mean(K.detach(), bc, stride)
    # the compressed branch's log-sum-exp; its output is not needed, V stands in for the pooled values
    _, lse = ops.attention_fwd(Q.detach(), K.detach(), K.detach(), branches=L.BRANCH_COMPRESSED, fused=False,
                               causal=bool(cfg.causal), scale=scale, Kc=Kc, Vc=Kc, cmp_block=bc, cmp_stride=stride,
                               cmp_offset=cmp_offset)
    return ops.cmp_block_scores(Q.detach(), Kc, lse, nk=nk, cmp_block=bc, cmp_stride=stride, cmp_offset=cmp_offset,
                                bn=int(cfg.block_size_n), sel_offset=sel_offset, causal=bool(cfg.causal), scale=scale,
                                force_first=int(getattr(cfg, "force_first", 0)), force_local=int(getattr(cfg, "force_local", 0)),
                                shared_per_group=bool(getattr(cfg, "select_per_group", False)))


def select_blocks_compressed(Q: Tensor, K: Tensor, cfg) -> Tensor:
    """int32 [B,H|Hkv,nq,min(top_k,nk)], descending score, ties to the lowest block index."""
    scores = compressed_block_scores(Q, K, cfg)
    _, _, _, _, sel_offset = _geometry(cfg, Q.shape[2], K.shape[2])
    return ops.topk_from_scores(scores, top_k=int(cfg.top_k), bm=int(cfg.block_size_m), bn=int(cfg.block_size_n),
                                offset=sel_offset, causal=bool(cfg.causal))


__all__ = ["compressed_block_scores", "select_blocks_compressed"]
