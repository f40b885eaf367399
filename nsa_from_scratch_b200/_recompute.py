"""Differentiable torch restatements of the compressed and sliding branches, used ONLY as
the backward of those two branches (the reference does the same through its plain-torch
functions, nsa/triton/forward.py:84-140,263-298).  Forward values never come from here.
Both run on the tensors' own device and keep memory at O(T*W) / O(T*Nc)."""
from __future__ import annotations

from typing import Optional

import torch
from torch import Tensor

from . import ops


def _expand_kv(x: Tensor, G: int) -> Tensor:
    return x if G == 1 else x.repeat_interleave(G, dim=1)


def _masked_attn(q: Tensor, k: Tensor, v: Tensor, mask: Tensor, s: float) -> Tensor:
    sc = torch.einsum("bhqd,bhkd->bhqk", q, k) * s
    sc = sc.masked_fill(~mask, float("-inf"))
    m = sc.amax(dim=-1, keepdim=True)
    m = torch.where(torch.isfinite(m), m, torch.zeros_like(m))
    p = torch.exp(sc - m)
    l = p.sum(-1, keepdim=True)
    return torch.einsum("bhqk,bhkd->bhqd", p / torch.where(l > 0, l, torch.ones_like(l)), v)


def compressed_torch(Q: Tensor, K: Tensor, V: Tensor, *, block_size_c: int, stride_c: Optional[int], causal: bool,
                     scale: Optional[float], chunk: int = 2048) -> Tensor:
    B, H, Tq, D = Q.shape
    Hkv, Tk = K.shape[1], K.shape[2]
    G = H // Hkv
    l = block_size_c
    d = l if stride_c is None else stride_c
    n = ops.n_pooled(Tk, l, d)
    s = ops.softmax_scale(D, scale)
    Kf, Vf = K.float(), V.float()
    if d == l:
        pad = n * l - Tk
        Kp = torch.nn.functional.pad(Kf, (0, 0, 0, pad)).view(B, Hkv, n, l, D).mean(3)
        Vp = torch.nn.functional.pad(Vf, (0, 0, 0, pad)).view(B, Hkv, n, l, D).mean(3)
        Tk_pad = n * l
    else:
        Kp = Kf.unfold(2, l, d)[:, :, :n].mean(-1)
        Vp = Vf.unfold(2, l, d)[:, :, :n].mean(-1)
        Tk_pad = Tk
    # the forward pooled in the input dtype; keep that rounding but pass gradients straight through
    Kp = Kp + (Kp.to(K.dtype).float() - Kp).detach()
    Vp = Vp + (Vp.to(V.dtype).float() - Vp).detach()
    Kp, Vp = _expand_kv(Kp, G), _expand_kv(Vp, G)
    outs = []
    c = torch.arange(n, device=Q.device).view(1, -1)
    for a in range(0, Tq, chunk):
        b = min(Tq, a + chunk)
        i = torch.arange(a, b, device=Q.device).view(-1, 1) + (Tk_pad - Tq)
        mask = (c * d + l - 1 <= i) if causal else torch.ones((b - a, n), dtype=torch.bool, device=Q.device)
        outs.append(_masked_attn(Q[:, :, a:b].float(), Kp, Vp, mask, s))
    return torch.cat(outs, dim=2)


def sliding_torch(Q: Tensor, K: Tensor, V: Tensor, *, window_size: int, causal: bool, scale: Optional[float]) -> Tensor:
    B, H, Tq, D = Q.shape
    Hkv, Tk = K.shape[1], K.shape[2]
    G = H // Hkv
    W = int(window_size)
    s = ops.softmax_scale(D, scale)
    off = Tk - Tq
    outs = []
    step = max(64, W)
    for a in range(0, Tq, step):
        b = min(Tq, a + step)
        lo = max(0, a + off - (W - 1 if causal else W))
        hi = max(lo, min(Tk, b + off + (0 if causal else W)))
        p = torch.arange(a, b, device=Q.device).view(-1, 1) + off
        j = torch.arange(lo, hi, device=Q.device).view(1, -1)
        mask = ((j <= p) & (j >= p - W + 1)) if causal else ((j <= p + W) & (j >= p - W))
        outs.append(_masked_attn(Q[:, :, a:b].float(), _expand_kv(K[:, :, lo:hi].float(), G),
                                 _expand_kv(V[:, :, lo:hi].float(), G), mask, s))
    return torch.cat(outs, dim=2)
