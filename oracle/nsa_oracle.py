"""CPU oracle for the Native-Sparse-Attention hot path.

TEST INFRASTRUCTURE ONLY.  This file is the checker that the CUDA kernels are
compared with; it is never the product.  Only the test-suite, the smoke check
and the CPU-baseline leg of the benchmark may import it.

It is an independent restatement (plain torch on CPU, fp32 internally) of the
algorithms in the reference project `qflen/nsa-from-scratch`:

* block mean pooling            nsa/triton/compressed.py:25-44, nsa/reference.py:94-108
* compressed attention          nsa/reference.py:71-134
* block scoring and top-k       nsa/triton/forward.py:321-359, nsa/reference.py:187-209,
                                nsa/triton/selected.py:153-185
* selected attention            nsa/reference.py:137-247, nsa/triton/selected.py:31-146
* sliding-window attention      nsa/reference.py:250-285
* gated combine                 nsa/triton/gating.py:15-40, nsa/reference.py:331-347
* selected backward             autograd through this file's selected attention
                                (what tests/test_selected_backward.py:73-126 does)
* fp8 quantise / dequantise     nsa/triton/fp8.py:20-40,67-69

Parity pin: `tests/golden/make_golden.py` runs the reference's own functions
and this restatement on the same seeded inputs and stores the reference's
outputs; `tests/test_oracle_golden.py` replays them.  Features the reference
does not have (grouped KV heads, stride < block pooling, forced blocks,
group-shared indices) are "parity unpinned": they are checked only through
the degenerate cases that collapse onto the pinned behaviour.

Differences in formulation from the reference (on purpose): attention is
evaluated as a masked dense softmax with an integer multiplicity matrix
instead of gather loops; grouped KV heads are indexed, never repeated; a
`rows=(q0, q1)` argument evaluates only a band of query rows against the full
key set so that 64k-token cases can be sampled in seconds.

Conventions (same as the reference): Q [B,H,Tq,D]; K,V [B,Hkv,Tk,D] with
H % Hkv == 0; queries align with the tail of the keys (offset = Tk - Tq);
lse is the natural-log sum-exp of the scaled scores, fp32 [B,H,Tq]; a row
with no legal key gives out = 0 and lse = -inf (the kernels' convention; the
reference's plain-torch functions give NaN there).
"""

from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
from torch import Tensor

NEG_INF = float("-inf")


# --------------------------------------------------------------------------
# helpers
# --------------------------------------------------------------------------

def _softmax_scale(D: int, scale: Optional[float]) -> float:
    return float(scale) if scale is not None else 1.0 / math.sqrt(D)


def _group(H: int, Hkv: int) -> int:
    assert H % Hkv == 0, "query heads must be a multiple of KV heads"
    return H // Hkv


def _masked_softmax_av(s: Tensor, w: Tensor, V: Tensor) -> Tuple[Tensor, Tensor]:
    """Weighted masked softmax.  s [..,M,N] fp32 scores, w [..,M,N] fp32 >= 0
    multiplicities (0 = masked), V [..,N,D].  Returns out [..,M,D], lse [..,M]."""
    s = torch.where(w > 0, s, torch.full_like(s, NEG_INF))
    m = s.max(dim=-1, keepdim=True).values
    m_safe = torch.where(torch.isfinite(m), m, torch.zeros_like(m))
    p = torch.exp(s - m_safe) * w
    l = p.sum(dim=-1, keepdim=True)
    ok = l > 0
    l_safe = torch.where(ok, l, torch.ones_like(l))
    out = torch.matmul(p / l_safe, V)
    lse = torch.where(ok, m_safe + torch.log(l_safe), torch.full_like(l, NEG_INF))
    return out, lse.squeeze(-1)


def _rows(rows: Optional[Tuple[int, int]], Tq: int) -> Tuple[int, int]:
    if rows is None:
        return 0, Tq
    q0, q1 = rows
    assert 0 <= q0 <= q1 <= Tq
    return q0, q1


# --------------------------------------------------------------------------
# pooling
# --------------------------------------------------------------------------

def pool_mean(x: Tensor, block: int, stride: Optional[int] = None) -> Tensor:
    """Mean over windows of `block` rows taken every `stride` rows, in x's dtype.

    stride None or == block restates the reference (compressed.py:25-44): the
    sequence is zero-padded to a multiple of `block`, so a trailing partial
    window is still divided by `block`.  stride < block (overlapping windows,
    parity unpinned) keeps only the windows that lie wholly inside the
    sequence: n_out = floor((T - block)/stride) + 1 (0 when T < block), no
    padding.

    Rounding points (they decide index parity, forward.py:338-347): fp32 sum
    of the `block` values, divide by `block`, one round-to-nearest-even to
    x.dtype.
    """
    B, H, T, D = x.shape
    stride = block if stride is None else stride
    assert 0 < stride <= block
    n_out = n_pooled(T, block, stride)
    Tp = n_out * block if stride == block else T
    if n_out == 0:
        return torch.zeros((B, H, 0, D), dtype=x.dtype)
    xf = torch.zeros((B, H, Tp, D), dtype=torch.float32)
    xf[:, :, :T] = x.float()
    win = xf.unfold(2, block, stride)[:, :, :n_out]          # [B,H,n_out,D,block]
    acc = torch.zeros((B, H, n_out, D), dtype=torch.float32)
    for r in range(block):                                     # sequential fp32 sum
        acc = acc + win[..., r]
    return (acc / float(block)).to(x.dtype)


def pool_learned(x: Tensor, proj: Tensor, block: int, stride: Optional[int] = None) -> Tensor:
    """fp32 [B,H,n,D]: window c = sum_s x[c*stride+s] * proj[s] (reference.py:109-113: zero padding to a multiple of
    the block, then einsum("bhnsd,sd->bhnd") over the block's rows); stride < block: whole windows only."""
    stride = block if stride is None else stride
    B, H, T, D = x.shape
    xf = x.float()
    if stride == block:
        n = (T + block - 1) // block
        xf = torch.nn.functional.pad(xf, (0, 0, 0, n * block - T))
        win = xf.view(B, H, n, block, D)
    else:
        win = xf.unfold(2, block, stride).permute(0, 1, 2, 4, 3) if T >= block else xf.new_zeros((B, H, 0, block, D))
    return torch.einsum("bhnsd,sd->bhnd", win, proj.float())


def n_pooled(T: int, block: int, stride: Optional[int] = None) -> int:
    stride = block if stride is None else stride
    if stride == block:
        return (T + block - 1) // block
    return (T - block) // stride + 1 if T >= block else 0


# --------------------------------------------------------------------------
# compressed branch
# --------------------------------------------------------------------------

def compressed_attention(
    Q: Tensor, K: Tensor, V: Tensor, *, block_size_c: int = 64,
    stride_c: Optional[int] = None, causal: bool = True,
    scale: Optional[float] = None, rows: Optional[Tuple[int, int]] = None,
    pool_proj_k: Optional[Tensor] = None, pool_proj_v: Optional[Tensor] = None,
) -> Tuple[Tensor, Tensor]:
    """Attention of Q over mean-pooled K/V (reference.py:71-134); with pool_proj_k / pool_proj_v
    [block_size_c, D] over learned-pooled K/V, sum_s K[c*stride+s] * proj[s] (reference.py:109-113).

    Causal rule (reference.py:122-126 with stride == block): pooled token c is
    visible to query row i iff its window ends at or before the query's key
    position, c*stride + block - 1 <= i + (Tk_padded - Tq).  With
    stride == block, Tk_padded is the key length zero-padded to a multiple of
    `block` -- the reference uses the PADDED length in the offset, reproduced
    here; with stride < block nothing is padded and Tk_padded = Tk.
    Returns fp32 out [B,H,R,D] and lse [B,H,R] for R = selected rows.
    """
    B, H, Tq, D = Q.shape
    Hkv, Tk = K.shape[1], K.shape[2]
    G = _group(H, Hkv)
    stride = block_size_c if stride_c is None else stride_c
    if pool_proj_k is not None:
        Kc = pool_learned(K, pool_proj_k, block_size_c, stride)
        Vc = pool_learned(V, pool_proj_v, block_size_c, stride)
    else:
        Kc = pool_mean(K, block_size_c, stride).float()
        Vc = pool_mean(V, block_size_c, stride).float()
    Nc = Kc.shape[2]
    Tk_pad = Nc * block_size_c if stride == block_size_c else Tk
    s = _softmax_scale(D, scale)
    q0, q1 = _rows(rows, Tq)
    i = torch.arange(q0, q1).view(-1, 1) + (Tk_pad - Tq)
    c = torch.arange(Nc).view(1, -1)
    if causal:
        w = (c * stride + block_size_c - 1 <= i).float()
    else:
        w = torch.ones((q1 - q0, Nc))
    out = torch.empty((B, H, q1 - q0, D), dtype=torch.float32)
    lse = torch.empty((B, H, q1 - q0), dtype=torch.float32)
    for h in range(H):
        sc = torch.matmul(Q[:, h, q0:q1].float(), Kc[:, h // G].transpose(-1, -2)) * s
        o, l = _masked_softmax_av(sc, w.expand_as(sc), Vc[:, h // G])
        out[:, h], lse[:, h] = o, l
    return out, lse


# --------------------------------------------------------------------------
# block scoring and top-k selection
# --------------------------------------------------------------------------

def block_scores(Q: Tensor, K: Tensor, *, block_size_m: int = 64, block_size_n: int = 64,
                 scale: Optional[float] = None, group_shared: bool = False) -> Tensor:
    """fp32 [B,H,nq,nk] scores: block means of Q and K taken in the input
    dtype, cast to fp32, dotted, times scale (forward.py:301-318,344-347).
    group_shared (parity unpinned): [B,Hkv,nq,nk]; the query vector of a KV
    head is the fp32 sum, in head order, of the block means of the query heads
    that share it."""
    B, H, Tq, D = Q.shape
    Hkv = K.shape[1]
    G = _group(H, Hkv)
    Qb = pool_mean(Q, block_size_m).float()
    Kb = pool_mean(K, block_size_n).float()
    if group_shared:
        Qg = Qb.view(B, Hkv, G, Qb.shape[2], D)
        qsum = Qg[:, :, 0].clone()
        for g in range(1, G):                       # fp32 sum of the heads' block means, in head order
            qsum = qsum + Qg[:, :, g]
        dots = torch.matmul(qsum, Kb.transpose(-1, -2))
    else:
        Kb = Kb.repeat_interleave(G, dim=1) if G > 1 else Kb
        dots = torch.matmul(Qb, Kb.transpose(-1, -2))
    return dots * _softmax_scale(D, scale)


def legal_blocks(nq: int, nk: int, bm: int, bn: int, offset: int) -> Tensor:
    """bool [nq,nk]: KV block c may be chosen by Q block q iff its first token
    is not after the Q block's last token, c*bn <= q*bm + bm-1 + offset
    (reference.py:196-206)."""
    q_last = torch.arange(nq).view(-1, 1) * bm + (bm - 1) + offset
    k_first = torch.arange(nk).view(1, -1) * bn
    return k_first <= q_last


def topk_canonical(scores: Tensor, top_k: int, *, legal: Optional[Tensor] = None,
                   force_first: int = 0, force_local: int = 0) -> Tensor:
    """int32 [..,nq,k] indices by descending score; ties (in particular the
    -inf slots of early Q blocks) resolved to the LOWEST block index.
    torch.topk (forward.py:357-359) leaves the order of tied slots
    unspecified; everywhere scores are distinct this equals it.

    force_first / force_local (parity unpinned): the first `force_first`
    blocks and the last `force_local` legal blocks of each row are given
    score +inf before sorting."""
    sc = scores.float().clone()
    nq, nk = sc.shape[-2], sc.shape[-1]
    if legal is not None:
        sc = sc.masked_fill(~legal.view((1,) * (sc.dim() - 2) + (nq, nk)), NEG_INF)
    if force_first or force_local:
        assert legal is not None
        c = torch.arange(nk).view(1, -1)
        last = legal.long().sum(-1, keepdim=True) - 1                       # [nq,1]
        forced = ((c < force_first) | ((c <= last) & (c > last - force_local))) & legal
        sc = sc.masked_fill(forced.view((1,) * (sc.dim() - 2) + (nq, nk)), float("inf"))
    k = min(top_k, nk)
    order = torch.sort(sc, dim=-1, descending=True, stable=True).indices
    return order[..., :k].to(torch.int32).contiguous()


def select_blocks(Q: Tensor, K: Tensor, *, block_size_m: int = 64, block_size_n: int = 64,
                  top_k: int = 16, causal: bool = True, scale: Optional[float] = None,
                  force_first: int = 0, force_local: int = 0, group_shared: bool = False,
                  return_scores: bool = False):
    """Indices the combined forward uses (forward.py:321-359).  The causal
    offset here is taken from the PADDED lengths, Tk_p - Tq_p (forward.py:350-352)."""
    Tq, Tk = Q.shape[2], K.shape[2]
    nq = (Tq + block_size_m - 1) // block_size_m
    nk = (Tk + block_size_n - 1) // block_size_n
    sc = block_scores(Q, K, block_size_m=block_size_m, block_size_n=block_size_n, scale=scale,
                      group_shared=group_shared)
    legal = None
    if causal:
        legal = legal_blocks(nq, nk, block_size_m, block_size_n,
                             nk * block_size_n - nq * block_size_m)
    elif force_first or force_local:
        legal = torch.ones((nq, nk), dtype=torch.bool)
    idx = topk_canonical(sc, top_k, legal=legal, force_first=force_first, force_local=force_local)
    if return_scores:
        masked = sc if legal is None else sc.masked_fill(~legal, NEG_INF)
        return idx, masked
    return idx


def moba_block_indices(Q: Tensor, K: Tensor, *, block_size_n: int = 64, block_size_m: int = 64,
                       top_k_per_query: int = 16, top_k_cap: int = 64, causal: bool = True,
                       scale: Optional[float] = None) -> Tensor:
    """MoBA routing as a producer of block lists (nsa/triton/moba.py:18-92): every query TOKEN takes its
    top_k_per_query key blocks by q . mean(K block) * scale (key block legal iff its first token is not after the
    token, offset from the PADDED lengths); a query block lists the union of its rows' picks in ascending order,
    padded with the out-of-range id nk up to cap = min(top_k_cap, nk); a union larger than the cap keeps the cap
    blocks with the best block-level score (max over the rows), best first.  Ties resolve to the lowest block id
    (torch.topk / argsort leave them unspecified).  A row with fewer legal blocks than picks contributes only its
    legal ones (the reference's top-k then returns arbitrary illegal ids, which its attention kernel skips).
    int32 [B,H,nq,cap]."""
    B, H, Tq, D = Q.shape
    Hkv, Tk = K.shape[1], K.shape[2]
    G = _group(H, Hkv)
    bn, bm = block_size_n, block_size_m
    nq, nk = (Tq + bm - 1) // bm, (Tk + bn - 1) // bn
    Kb = pool_mean(K, bn).float()
    Qp = torch.nn.functional.pad(Q.float(), (0, 0, 0, nq * bm - Tq))
    s = _softmax_scale(D, scale)
    offset = nk * bn - nq * bm
    rows = torch.arange(nq * bm).view(-1, 1)
    legal = (torch.arange(nk).view(1, -1) * bn <= rows + offset) if causal else torch.ones((nq * bm, nk), dtype=torch.bool)
    kq = min(top_k_per_query, nk)
    cap = min(top_k_cap, nk)
    out = torch.full((B, H, nq, cap), nk, dtype=torch.int32)
    for b in range(B):
        for h in range(H):
            sc = torch.matmul(Qp[b, h], Kb[b, h // G].t()) * s
            sc = sc.masked_fill(~legal, NEG_INF)
            order = torch.sort(sc, dim=-1, descending=True, stable=True).indices[:, :kq]      # ties -> lowest id
            level = sc.view(nq, bm, nk).amax(dim=1)
            took = torch.gather(sc, 1, order) > NEG_INF              # a row with fewer legal blocks than picks: the rest is dropped
            picks = torch.where(took, order, torch.full_like(order, nk)).reshape(nq, bm * kq)
            for qb in range(nq):
                u = torch.unique(picks[qb])
                u = u[u < nk]
                if u.numel() > cap:
                    keep = torch.sort(level[qb][u], descending=True, stable=True).indices[:cap]
                    u = u[keep]
                out[b, h, qb, : u.numel()] = u.to(torch.int32)
    return out


def overlap_weights(n_cmp: int, nk: int, block_size_c: int, stride_c: int, block_size_n: int) -> Tensor:
    """fp32 [n_cmp, nk]: share of compressed token c's window [c*stride, c*stride + block_c) that lies in
    selection block j = [j*bn, (j+1)*bn), i.e. |overlap| / block_c (exact in fp32 for power-of-two sizes)."""
    c0 = torch.arange(n_cmp).view(-1, 1) * stride_c
    j0 = torch.arange(nk).view(1, -1) * block_size_n
    ov = (torch.minimum(c0 + block_size_c, j0 + block_size_n) - torch.maximum(c0, j0)).clamp(min=0)
    return ov.float() / float(block_size_c)


def compressed_block_scores(Q: Tensor, K: Tensor, *, block_size_c: int = 32, stride_c: Optional[int] = None,
                            block_size_m: int = 64, block_size_n: int = 64, causal: bool = True,
                            scale: Optional[float] = None, group_shared: bool = False) -> Tensor:
    """Selection scores taken from the compressed branch's attention probabilities (the scorer of the NSA
    paper; parity unpinned -- the reference scores with block means, forward.py:321-359).
    p[i,c] = softmax over the compressed tokens visible to row i of (q_i . Kc_c) * scale -- the
    probabilities `compressed_attention` uses; a compressed token hands its probability to the selection
    blocks its window overlaps, in proportion to the overlap (`overlap_weights`); the score of (query
    block, selection block) is the sum over the query block's rows -- and, group_shared, over the
    query heads of the KV head.  fp32 [B,H|Hkv,nq,nk]."""
    B, H, Tq, D = Q.shape
    Hkv, Tk = K.shape[1], K.shape[2]
    G = _group(H, Hkv)
    stride = block_size_c if stride_c is None else stride_c
    Kc = pool_mean(K, block_size_c, stride).float()
    Nc = Kc.shape[2]
    Tk_pad = Nc * block_size_c if stride == block_size_c else Tk
    s = _softmax_scale(D, scale)
    nq = (Tq + block_size_m - 1) // block_size_m
    nk = (Tk + block_size_n - 1) // block_size_n
    W = overlap_weights(Nc, nk, block_size_c, stride, block_size_n)
    i = torch.arange(Tq).view(-1, 1) + (Tk_pad - Tq)
    c = torch.arange(Nc).view(1, -1)
    vis = (c * stride + block_size_c - 1 <= i) if causal else torch.ones((Tq, Nc), dtype=torch.bool)
    out = torch.zeros((B, H, nq, nk), dtype=torch.float32)
    for h in range(H):
        sc = torch.matmul(Q[:, h].float(), Kc[:, h // G].transpose(-1, -2)) * s
        sc = sc.masked_fill(~vis, NEG_INF)
        p = torch.softmax(sc, dim=-1)
        p = torch.where(vis.any(-1, keepdim=True), p, torch.zeros_like(p))      # rows without a visible token
        ps = torch.matmul(p, W)                                                  # [B,Tq,nk]
        pad = nq * block_size_m - Tq
        if pad:
            ps = torch.nn.functional.pad(ps, (0, 0, 0, pad))
        out[:, h] = ps.view(B, nq, block_size_m, nk).sum(2)
    if group_shared:
        out = out.view(B, Hkv, G, nq, nk).sum(2)
    return out


def indices_from_scores(scores: Tensor, *, top_k: int, block_size_m: int, block_size_n: int,
                        Tq: int, Tk: int, causal: bool) -> Tensor:
    """Indices from caller-supplied scores (selected.py:153-185); here the
    offset is the UNPADDED Tk - Tq."""
    nq, nk = scores.shape[-2], scores.shape[-1]
    legal = legal_blocks(nq, nk, block_size_m, block_size_n, Tk - Tq) if causal else None
    return topk_canonical(scores, top_k, legal=legal)


# --------------------------------------------------------------------------
# selected branch
# --------------------------------------------------------------------------

def _selection_weights(idx_row: Tensor, nk: int, bn: int) -> Tensor:
    """idx_row [k] -> fp32 [nk*bn] token multiplicities.  A block listed twice
    counts twice (moba.py:78-82); ids outside [0,nk) are skipped."""
    ok = (idx_row >= 0) & (idx_row < nk)
    cnt = torch.zeros(nk, dtype=torch.float32)
    cnt.index_add_(0, idx_row[ok].long(), torch.ones(int(ok.sum()), dtype=torch.float32))
    return cnt.repeat_interleave(bn)


def selected_attention(
    Q: Tensor, K: Tensor, V: Tensor, block_indices: Tensor, *, block_size_n: int = 64,
    block_size_m: int = 64, causal: bool = True, scale: Optional[float] = None,
    rows: Optional[Tuple[int, int]] = None,
) -> Tuple[Tensor, Tensor]:
    """Attention of each Q block over its listed KV blocks (reference.py:211-247,
    selected.py:83-140).  block_indices [B,H|Hkv,nq,k].  K/V are zero-padded to
    a multiple of block_size_n and the padded keys are attendable unless the
    causal rule j <= i + (Tk - Tq) (UNPADDED offset, selected.py:300) hides
    them.  Differentiable.  Returns fp32 out [B,H,R,D], lse [B,H,R]."""
    B, H, Tq, D = Q.shape
    Hkv, Tk = K.shape[1], K.shape[2]
    G = _group(H, Hkv)
    bn, bm = block_size_n, block_size_m
    nk = (Tk + bn - 1) // bn
    nq = (Tq + bm - 1) // bm
    Hi = block_indices.shape[1]
    assert Hi in (H, Hkv) and block_indices.shape[2] == nq
    Kp = torch.nn.functional.pad(K.float(), (0, 0, 0, nk * bn - Tk))
    Vp = torch.nn.functional.pad(V.float(), (0, 0, 0, nk * bn - Tk))
    s = _softmax_scale(D, scale)
    q0, q1 = _rows(rows, Tq)
    j = torch.arange(nk * bn).view(1, -1)
    outs, lses = [], []
    for b in range(B):
        ob, lb = [], []
        for h in range(H):
            hi = h if Hi == H else h // G
            o_rows, l_rows = [], []
            qb0, qb1 = q0 // bm, (q1 + bm - 1) // bm if q1 > q0 else q0 // bm
            for qb in range(qb0, qb1):
                r0, r1 = max(q0, qb * bm), min(q1, (qb + 1) * bm, Tq)
                if r1 <= r0:
                    continue
                w = _selection_weights(block_indices[b, hi, qb], nk, bn).view(1, -1)
                w = w.expand(r1 - r0, -1)
                if causal:
                    i = torch.arange(r0, r1).view(-1, 1) + (Tk - Tq)
                    w = w * (j <= i).float()
                sc = torch.matmul(Q[b, h, r0:r1].float(), Kp[b, h // G].t()) * s
                o, l = _masked_softmax_av(sc, w, Vp[b, h // G])
                o_rows.append(o)
                l_rows.append(l)
            ob.append(torch.cat(o_rows, 0) if o_rows else torch.zeros((0, D)))
            lb.append(torch.cat(l_rows, 0) if l_rows else torch.zeros((0,)))
        outs.append(torch.stack(ob, 0))
        lses.append(torch.stack(lb, 0))
    return torch.stack(outs, 0), torch.stack(lses, 0)


def selected_backward(
    dO: Tensor, Q: Tensor, K: Tensor, V: Tensor, block_indices: Tensor, *,
    block_size_n: int = 64, block_size_m: int = 64, causal: bool = True,
    scale: Optional[float] = None,
) -> Tuple[Tensor, Tensor, Tensor]:
    """fp32 dQ [B,H,Tq,D], dK, dV [B,Hkv,Tk,D] by autograd through
    `selected_attention` (the reference's own acceptance test does the same
    through its plain-torch function, tests/test_selected_backward.py:95-115).
    Rows without a legal key contribute nothing."""
    Qd = Q.detach().float().requires_grad_(True)
    Kd = K.detach().float().requires_grad_(True)
    Vd = V.detach().float().requires_grad_(True)
    out, _ = selected_attention(Qd, Kd, Vd, block_indices, block_size_n=block_size_n,
                                block_size_m=block_size_m, causal=causal, scale=scale)
    dQ, dK, dV = torch.autograd.grad(out, (Qd, Kd, Vd), grad_outputs=dO.float(),
                                     allow_unused=True)
    z = lambda g, x: torch.zeros_like(x) if g is None else torch.nan_to_num(g, 0.0, 0.0, 0.0)
    return z(dQ, Qd), z(dK, Kd), z(dV, Vd)


def branch_backward(kind: str, dO: Tensor, Q: Tensor, K: Tensor, V: Tensor, **kw) -> Tuple[Tensor, Tensor, Tensor]:
    """fp32 (dQ, dK, dV) of the compressed ("cmp") or sliding ("sld") branch by autograd through this
    file's forward -- the reference's own backward for these branches is autograd through its
    plain-torch functions with NaN rows zeroed (nsa/triton/forward.py:84-120,133-140,273-298)."""
    Qd, Kd, Vd = (t.detach().float().requires_grad_(True) for t in (Q, K, V))
    fn = compressed_attention if kind == "cmp" else sliding_attention
    out, _ = fn(Qd, Kd, Vd, **kw)
    grads = torch.autograd.grad(out, (Qd, Kd, Vd), grad_outputs=dO.float(), allow_unused=True)
    return tuple(torch.zeros_like(x) if g is None else torch.nan_to_num(g, 0.0, 0.0, 0.0)
                 for g, x in zip(grads, (Qd, Kd, Vd)))


# --------------------------------------------------------------------------
# sliding-window branch
# --------------------------------------------------------------------------

def sliding_attention(
    Q: Tensor, K: Tensor, V: Tensor, *, window_size: int = 512, causal: bool = True,
    scale: Optional[float] = None, rows: Optional[Tuple[int, int]] = None,
) -> Tuple[Tensor, Tensor]:
    """Causal: keys j in [p-W+1, p] with p = i + (Tk - Tq); symmetric:
    |j - p| <= W (reference.py:273-279).  Only the band of keys a row block can
    see is touched, so 64k-token cases stay cheap."""
    B, H, Tq, D = Q.shape
    Hkv, Tk = K.shape[1], K.shape[2]
    G = _group(H, Hkv)
    W = int(window_size)
    s = _softmax_scale(D, scale)
    q0, q1 = _rows(rows, Tq)
    off = Tk - Tq
    out = torch.zeros((B, H, q1 - q0, D), dtype=torch.float32)
    lse = torch.full((B, H, q1 - q0), NEG_INF, dtype=torch.float32)
    step = max(64, W)
    for a in range(q0, q1, step):
        b_ = min(q1, a + step)
        lo = max(0, a + off - (W - 1 if causal else W))
        hi = min(Tk, b_ + off + (0 if causal else W))
        if hi <= lo:
            continue
        p = torch.arange(a, b_).view(-1, 1) + off
        j = torch.arange(lo, hi).view(1, -1)
        w = ((j <= p) & (j >= p - W + 1)) if causal else ((j <= p + W) & (j >= p - W))
        w = w.float()
        for h in range(H):
            sc = torch.matmul(Q[:, h, a:b_].float(), K[:, h // G, lo:hi].float().transpose(-1, -2)) * s
            o, l = _masked_softmax_av(sc, w.expand_as(sc), V[:, h // G, lo:hi].float())
            out[:, h, a - q0:b_ - q0], lse[:, h, a - q0:b_ - q0] = o, l
    return out, lse


# --------------------------------------------------------------------------
# gates and the combined forward
# --------------------------------------------------------------------------

def gate_values(gate_logits: Tensor, activation: str = "sigmoid") -> Tensor:
    if activation == "sigmoid":
        return torch.sigmoid(gate_logits)
    if activation == "softmax":
        return torch.softmax(gate_logits, dim=-1)
    raise ValueError(f"unknown activation: {activation}")


def combine(out_c: Tensor, out_s: Tensor, out_w: Tensor, gate_logits: Tensor,
            activation: str = "sigmoid") -> Tensor:
    """g0*out_c + g1*out_s + g2*out_w evaluated left to right in the tensors'
    own dtypes with torch's promotion rules (gating.py:34-40): with bf16
    operands every product and every sum is rounded to bf16."""
    g = gate_values(gate_logits, activation)
    return g[..., 0:1] * out_c + g[..., 1:2] * out_s + g[..., 2:3] * out_w


def nsa_forward(
    Q: Tensor, K: Tensor, V: Tensor, *, block_size_c: int = 64, stride_c: Optional[int] = None,
    block_size_n: int = 64, block_size_m: int = 64, top_k: int = 16, window_size: int = 512,
    causal: bool = True, scale: Optional[float] = None, gate_logits: Optional[Tensor] = None,
    gate_activation: str = "sigmoid", block_indices: Optional[Tensor] = None,
    force_first: int = 0, force_local: int = 0, group_shared: bool = False,
    rows: Optional[Tuple[int, int]] = None,
    pool_proj_k: Optional[Tensor] = None, pool_proj_v: Optional[Tensor] = None,
) -> Tensor:
    """fp32 combined forward (forward.py:362-406 / reference.py:288-347): the
    three branches on the same inputs, gates applied in fp32.  With
    block_indices None the indices come from `select_blocks`."""
    B, H, Tq, D = Q.shape
    if block_indices is None:
        block_indices = select_blocks(Q, K, block_size_m=block_size_m, block_size_n=block_size_n,
                                      top_k=top_k, causal=causal, scale=scale,
                                      force_first=force_first, force_local=force_local,
                                      group_shared=group_shared)
    q0, q1 = _rows(rows, Tq)
    oc, _ = compressed_attention(Q, K, V, block_size_c=block_size_c, stride_c=stride_c,
                                 causal=causal, scale=scale, rows=(q0, q1),
                                 pool_proj_k=pool_proj_k, pool_proj_v=pool_proj_v)
    os_, _ = selected_attention(Q, K, V, block_indices, block_size_n=block_size_n,
                                block_size_m=block_size_m, causal=causal, scale=scale,
                                rows=(q0, q1))
    ow, _ = sliding_attention(Q, K, V, window_size=window_size, causal=causal, scale=scale,
                              rows=(q0, q1))
    if gate_logits is None:
        g = torch.full((B, H, q1 - q0, 3), 0.5 if gate_activation == "sigmoid" else 1.0 / 3.0)
    else:
        g = gate_values(gate_logits[:, :, q0:q1].float(), gate_activation)
    return g[..., 0:1] * oc + g[..., 1:2] * os_ + g[..., 2:3] * ow


# --------------------------------------------------------------------------
# fp8 storage path
# --------------------------------------------------------------------------

_FP8_MAX = {torch.float8_e4m3fn: 448.0, torch.float8_e5m2: 57344.0}


def rope(x: Tensor, cos: Tensor, sin: Tensor) -> Tensor:
    """Rotary embedding of a head-major tensor x [B,H,T,D] with tables [T,D], fp32:
    x*cos + rotate_half(x)*sin, rotate_half(x) = (-x[D/2:], x[:D/2])
    (nsa/model/llama_dense.py:19-37)."""
    x = x.float()
    h = x.shape[-1] // 2
    rot = torch.cat((-x[..., h:], x[..., :h]), dim=-1)
    return x * cos.float()[None, None] + rot * sin.float()[None, None]


def attention_layer(x: Tensor, w: dict, cos: Tensor, sin: Tensor, *, n_heads: int, head_dim: int,
                    n_kv_heads: Optional[int] = None, round_to: Optional[torch.dtype] = None, **nsa_kw) -> Tensor:
    """The attention module around the combined forward (nsa/model/llama_nsa.py:67-96), fp32:
    q/k/v/gate projections of x [B,T,hidden], rotary embedding of q and k, `nsa_forward`, the
    transpose back to [B,T,H*D] and the output projection.  `w` holds q_proj/k_proj/v_proj/o_proj/gate
    `.weight` tensors.  `round_to` rounds q, k, v (after the rotary embedding) to a 16-bit type and back,
    as a 16-bit kernel path sees them."""
    B, T, _ = x.shape
    H, D = n_heads, head_dim
    Hkv = H if n_kv_heads is None else n_kv_heads
    x = x.float()
    q = (x @ w["q_proj.weight"].float().T).view(B, T, H, D).transpose(1, 2)
    k = (x @ w["k_proj.weight"].float().T).view(B, T, Hkv, D).transpose(1, 2)
    v = (x @ w["v_proj.weight"].float().T).view(B, T, Hkv, D).transpose(1, 2)
    q, k = rope(q, cos, sin), rope(k, cos, sin)
    if round_to is not None:
        q, k, v = (t.to(round_to).float() for t in (q, k, v))
    gates = (x @ w["gate.weight"].float().T).view(B, T, H, 3).permute(0, 2, 1, 3)
    out = nsa_forward(q, k, v, gate_logits=gates, **nsa_kw)
    out = out.transpose(1, 2).reshape(B, T, H * D)
    return out @ w["o_proj.weight"].float().T


def quantize_to_fp8(x: Tensor, *, fmt: torch.dtype = torch.float8_e4m3fn,
                    eps: float = 1e-12) -> Tuple[Tensor, float]:
    """Per-tensor absmax quantisation (fp8.py:20-40): scale = absmax/fmt_max;
    x/scale is evaluated in x's dtype (so a bf16 input is rounded to bf16
    before the saturating cast)."""
    fmax = _FP8_MAX[fmt]
    absmax = float(x.detach().abs().max().clamp(min=eps))
    scale = absmax / fmax
    return (x / scale).clamp(-fmax, fmax).to(fmt), scale


def dequantize_fp8(x8: Tensor, scale: float) -> Tensor:
    """bf16(fp32(x8) * fp32(scale)), the operands the fp8 wrapper feeds the
    bf16 kernel (fp8.py:67-69)."""
    return x8.to(torch.bfloat16) * scale


# --------------------------------------------------------------------------
# algorithmic work (for roofline figures)
# --------------------------------------------------------------------------

def pair_counts(T: int, *, block_size_c: int, stride_c: int, window: int,
                block_indices_row_heads: Optional[Tensor] = None, bn: int = 64, bm: int = 64):
    """Unmasked (q,k) pairs per head for causal Tq == Tk == T: returns
    (compressed, sliding, selected-or-None).  selected is summed over the
    heads present in `block_indices_row_heads` [Hn,nq,k]."""
    t = torch.arange(T, dtype=torch.int64)
    Tk_pad = T if stride_c != block_size_c else (-(-T // block_size_c)) * block_size_c
    n_c = n_pooled(T, block_size_c, stride_c)
    vis = torch.clamp((t + (Tk_pad - T) - (block_size_c - 1)) // stride_c + 1, min=0, max=n_c)
    vis = torch.where(t + (Tk_pad - T) - (block_size_c - 1) >= 0, vis, torch.zeros_like(vis))
    cmp_pairs = int(vis.sum())
    sld_pairs = int(torch.clamp(t + 1, max=window).sum())
    sel_pairs = None
    if block_indices_row_heads is not None:
        idx = block_indices_row_heads.long()
        Hn, nq, k = idx.shape
        nk = -(-T // bn)
        qb = torch.arange(nq).view(1, nq, 1)
        ok = (idx >= 0) & (idx < nk)
        # rows r of q block qb see tokens j of block c with j <= r: full if c < qb, triangle if c == qb
        rows_in_block = torch.clamp(torch.tensor(T) - qb * bm, max=bm)
        full = (idx < qb) & ok
        diag = (idx == qb) & ok
        tri = rows_in_block * (rows_in_block + 1) // 2
        sel_pairs = int((full * (rows_in_block * bn)).sum() + (diag * tri).sum())
    return cmp_pairs, sld_pairs, sel_pairs
