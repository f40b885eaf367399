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


def forward_with_compressed_scorer(Q: Tensor, K: Tensor, V: Tensor, cfg, gate_logits=None) -> Tensor:
    """The combined forward when the selection depends on the compressed branch: the compressed branch runs first
    (gated result into the output, its lse kept), the scores and indices follow from that lse, then the selected
    and sliding branches are added to the same output rows.  Nothing is computed twice.  Inference route (the
    differentiable route takes the indices from `select_blocks_compressed` and runs the branches separately)."""
    B, H, Tq, D = Q.shape
    Tk = K.shape[2]
    scale = float(cfg.scale if cfg.scale is not None else 1.0 / (D ** 0.5))
    bc, stride, cmp_offset, nk, sel_offset = _geometry(cfg, Tq, Tk)
    act = L.GATE_SOFTMAX if cfg.gate_activation == "softmax" else L.GATE_SIGMOID
    Kc, Vc = ops.pool_mean(K, bc, stride), ops.pool_mean(V, bc, stride)
    # launches that add to an existing output exist on the tcgen05 kernel only; other shapes select, then run the
    # ordinary single-launch forward
    if not (D in (64, 128) and int(cfg.block_size_m) == 64 and int(cfg.block_size_n) == 64 and int(cfg.top_k) <= 64
            and ops.engine() != L.ENGINE_GENERIC):
        from .forward import _fused_forward
        return _fused_forward(Q, K, V, cfg, scale, getattr(cfg, "stride_c", None), gate_logits,
                              select_blocks_compressed(Q, K, cfg), 1.0, 1.0, 1.0)
    out, lse = ops.attention_fwd(Q, K, V, branches=L.BRANCH_COMPRESSED, fused=True, fused_lse=True, causal=bool(cfg.causal),
                                 scale=scale, Kc=Kc, Vc=Vc, cmp_block=bc, cmp_stride=stride, cmp_offset=cmp_offset,
                                 gates=gate_logits, gate_act=act)
    scores = ops.cmp_block_scores(Q, Kc, lse, nk=nk, cmp_block=bc, cmp_stride=stride, cmp_offset=cmp_offset,
                                  bn=int(cfg.block_size_n), sel_offset=sel_offset, causal=bool(cfg.causal), scale=scale,
                                  force_first=int(getattr(cfg, "force_first", 0)), force_local=int(getattr(cfg, "force_local", 0)),
                                  shared_per_group=bool(getattr(cfg, "select_per_group", False)))
    idx = ops.topk_from_scores(scores, top_k=int(cfg.top_k), bm=int(cfg.block_size_m), bn=int(cfg.block_size_n),
                               offset=sel_offset, causal=bool(cfg.causal))
    ops.attention_fwd(Q, K, V, branches=L.BRANCH_SELECTED | L.BRANCH_SLIDING, fused=True, causal=bool(cfg.causal), scale=scale,
                      idx=idx, bm=int(cfg.block_size_m), bn=int(cfg.block_size_n), window=cfg.window_size, gates=gate_logits,
                      gate_act=act, accumulate_into=out)
    return out


__all__ = ["compressed_block_scores", "select_blocks_compressed", "forward_with_compressed_scorer"]
