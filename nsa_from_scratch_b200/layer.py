"""The caller of the NSA forward: the attention module between its projections.

Mirrors `NSAAttention.forward` of the reference (nsa/model/llama_nsa.py:67-96):

    q,k,v = proj(x).view(B,T,H,D).transpose(1,2); q,k = rope(q,k); gates = gate(x).view(B,T,H,3).permute(0,2,1,3)
    out = nsa_forward(q,k,v,cfg,gate_logits=gates); out = out.transpose(1,2).contiguous().view(B,T,H*D)

Between the projection GEMMs and `o_proj` the reference makes ten full-tensor passes (three transposes
to head-major, five element-wise kernels of the rotary embedding, the bf16 casts, the gate permute and
the transpose back).  Here each of q, k, v is read once and written once by `nsa_rope_to_heads`
(rotation in fp32, one rounding, head-major 16-bit result), the gate logits are read where they lie
([B,T,H,3]) and the kernel writes [B,T,H*D] directly.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn
from torch import Tensor

from . import ops
from .forward import _cfg, _fused_forward, _resolve_block_indices, nsa_forward


def rope_cache(seq_len: int, head_dim: int, base: float, device, dtype=torch.float32):
    """cos/sin tables [T, D] (`_build_rope_cache`, nsa/model/llama_dense.py:24-29)."""
    inv_freq = 1.0 / (base ** (torch.arange(0, head_dim, 2, device=device, dtype=torch.float32) / head_dim))
    t = torch.arange(seq_len, device=device, dtype=torch.float32)
    emb = torch.outer(t, inv_freq)
    emb = torch.cat((emb, emb), dim=-1)
    return emb.cos().to(dtype), emb.sin().to(dtype)


def nsa_attention_token_major(q: Tensor, k: Tensor, v: Tensor, cos: Optional[Tensor], sin: Optional[Tensor], cfg, *,
                              gate_logits: Optional[Tensor] = None, dtype: torch.dtype = torch.bfloat16,
                              pool_proj_k: Optional[Tensor] = None, pool_proj_v: Optional[Tensor] = None) -> Tensor:
    """q [B,T,H,D], k/v [B,T,Hkv,D] as the projections leave them (fp32, bf16 or fp16), cos/sin [T,D]
    (None: no rotary embedding), gate_logits [B,T,H,3] -> [B,T,H*D] in `dtype`.  Inference path (no autograd).
    pool_proj_k / pool_proj_v [block_size_c, D]: learned pooling (cfg.pool == "learned")."""
    B, T, H, D = q.shape
    qh = ops.rope_to_heads(q, cos, sin, dtype)
    kh = ops.rope_to_heads(k, cos, sin, dtype)
    vh = ops.rope_to_heads(v, None, None, dtype)
    scale = cfg.scale if cfg.scale is not None else 1.0 / (D ** 0.5)
    idx = _resolve_block_indices(qh, kh, block_size_m=cfg.block_size_m, block_size_n=cfg.block_size_n, top_k=cfg.top_k,
                                 causal=cfg.causal, scale=float(scale), force_first=_cfg(cfg, "force_first", 0),
                                 force_local=_cfg(cfg, "force_local", 0),
                                 shared_per_group=bool(_cfg(cfg, "select_per_group", False)))
    learned = getattr(cfg, "pool", "mean") == "learned"
    if learned and (pool_proj_k is None or pool_proj_v is None):
        raise ValueError("pool='learned' needs pool_proj_k and pool_proj_v")
    out = _fused_forward(qh, kh, vh, cfg, float(scale), getattr(cfg, "stride_c", None), gate_logits, idx, 1.0, 1.0, 1.0,
                         token_major=True, pool_proj=(pool_proj_k, pool_proj_v) if learned else None)
    return out.view(B, T, H * D)


class NSAAttention(nn.Module):
    """Same parameters and forward signature as the reference's module (nsa/model/llama_nsa.py:38-96), so a
    state dict moves across unchanged; `n_kv_heads` < `n_heads` (grouped K/V) is an extension.
    Without autograd the token-major route above runs; with it, the reference's own sequence of
    steps around the differentiable `nsa_forward`."""

    def __init__(self, hidden_size: int, n_heads: int, head_dim: int, nsa_cfg, n_kv_heads: Optional[int] = None):
        super().__init__()
        self.n_heads, self.head_dim = n_heads, head_dim
        self.n_kv_heads = n_heads if n_kv_heads is None else n_kv_heads
        self.nsa_cfg = nsa_cfg
        # learned compressed-pool projections, as the reference module creates them (nsa/model/llama_nsa.py:59-65);
        # used by the inference route only -- training with pool="learned" is not provided
        if getattr(nsa_cfg, "pool", "mean") == "learned":
            self.pool_proj_k = nn.Parameter(torch.randn(int(nsa_cfg.block_size_c), head_dim) / head_dim ** 0.5)
            self.pool_proj_v = nn.Parameter(torch.randn(int(nsa_cfg.block_size_c), head_dim) / head_dim ** 0.5)
        else:
            self.pool_proj_k = self.pool_proj_v = None
        self.q_proj = nn.Linear(hidden_size, n_heads * head_dim, bias=False)
        self.k_proj = nn.Linear(hidden_size, self.n_kv_heads * head_dim, bias=False)
        self.v_proj = nn.Linear(hidden_size, self.n_kv_heads * head_dim, bias=False)
        self.o_proj = nn.Linear(n_heads * head_dim, hidden_size, bias=False)
        self.gate = nn.Linear(hidden_size, n_heads * 3, bias=False)

    def forward(self, x: Tensor, cos: Tensor, sin: Tensor) -> Tensor:
        B, T, _ = x.shape
        H, Hkv, D = self.n_heads, self.n_kv_heads, self.head_dim
        q = self.q_proj(x).view(B, T, H, D)
        k = self.k_proj(x).view(B, T, Hkv, D)
        v = self.v_proj(x).view(B, T, Hkv, D)
        gates = self.gate(x).view(B, T, H, 3)
        if not (torch.is_grad_enabled() and (x.requires_grad or any(p.requires_grad for p in self.parameters()))):
            out = nsa_attention_token_major(q, k, v, cos, sin, self.nsa_cfg, gate_logits=gates, pool_proj_k=self.pool_proj_k,
                                            pool_proj_v=self.pool_proj_v).to(x.dtype)
            return self.o_proj(out)
        q, k, v = (t.transpose(1, 2) for t in (q, k, v))
        c, s = cos[None, None], sin[None, None]
        rot = lambda t: torch.cat((-t[..., D // 2:], t[..., :D // 2]), dim=-1)
        q, k = q * c + rot(q) * s, k * c + rot(k) * s
        kd = torch.bfloat16
        out = nsa_forward(q.to(kd), k.to(kd), v.to(kd), self.nsa_cfg,
                          gate_logits=gates.permute(0, 2, 1, 3).contiguous().to(kd)).to(x.dtype)
        return self.o_proj(out.transpose(1, 2).contiguous().view(B, T, H * D))


__all__ = ["NSAAttention", "nsa_attention_token_major", "rope_cache"]
