"""Combined NSA forward.  Same entry points as the reference's nsa/triton/forward.py:
`nsa_forward` (:362-370), `_resolve_block_indices` (:321-324), `_block_scores_from_pooled`
(:301-303) and the autograd Functions `_CompressedFn/_SelectedFn/_SlidingFn` (:123,143,263).

Without autograd the whole forward is four launches: pool K/V, pool Q/K block means,
score+top-k, and ONE fused kernel that runs the three branches per query tile and applies
the gates in its epilogue (no branch output ever reaches HBM).  With autograd the branches
run separately so that their outputs and log-sum-exps can be saved; every branch has a
hand-written backward kernel (the reference differentiates its plain-torch functions for the
compressed and sliding branches, nsa/triton/forward.py:133-140,273-298)."""
from __future__ import annotations

from typing import Optional

import torch
from torch import Tensor

from . import _lib as L
from . import ops
from .compressed import compressed_attention as _compressed_kernel
from .gating import combine
from .selected import selected_attention as _selected_kernel
from .sliding import sliding_attention as _sliding_kernel


def _block_scores_from_pooled(Q: Tensor, K: Tensor, *, block_size_m: int, block_size_n: int, scale: float) -> Tensor:
    """fp32 [B,H,nq,nk]: block means in the input dtype (pool kernel), then a library GEMM."""
    G = Q.shape[1] // K.shape[1]
    Qb = ops.pool_mean(Q, block_size_m).float()
    Kb = ops.pool_mean(K, block_size_n).float()
    Kb = Kb if G == 1 else Kb.repeat_interleave(G, dim=1)
    return torch.einsum("bhqd,bhkd->bhqk", Qb, Kb) * scale


def _resolve_block_indices(Q: Tensor, K: Tensor, *, block_size_m: int, block_size_n: int, top_k: int, causal: bool,
                           scale: float, force_first: int = 0, force_local: int = 0,
                           q_scale: float = 1.0, k_scale: float = 1.0, shared_per_group: bool = False) -> Tensor:
    """int32 [B,H,nq,min(top_k,nk)] by mean-pool scoring + top-k, ties to the lowest index.
    The causal legality offset uses the PADDED lengths, as the reference does (:350-352).
    shared_per_group: one row per KV head, [B,Hkv,nq,k], scored by the sum of its query heads' scores."""
    Tq, Tk = Q.shape[2], K.shape[2]
    Qb = ops.pool_mean(Q.detach(), block_size_m, dequant_scale=q_scale)
    Kb = ops.pool_mean(K.detach(), block_size_n, dequant_scale=k_scale)
    nq, nk = Qb.shape[2], Kb.shape[2]
    return ops.select_blocks_from_means(Qb, Kb, top_k=top_k, bm=block_size_m, bn=block_size_n,
                                        offset=nk * block_size_n - nq * block_size_m, causal=bool(causal),
                                        scale=float(scale), force_first=force_first, force_local=force_local,
                                        shared_per_group=shared_per_group)


class _CompressedFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, Q, K, V, block_size_c, pool, causal, scale, stride_c=None):
        out, lse = _compressed_kernel(Q, K, V, block_size_c=block_size_c, pool=pool, causal=causal, scale=scale,
                                      stride_c=stride_c)
        ctx.save_for_backward(Q, K, V, out, lse)
        ctx.args = (block_size_c, stride_c, causal, scale)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        Q, K, V, O, LSE = ctx.saved_tensors
        bc, sc, causal, scale = ctx.args
        D, Tq, Tk = Q.shape[-1], Q.shape[2], K.shape[2]
        stride = bc if sc is None else int(sc)
        Kc, Vc = ops.pool_mean(K, bc, stride), ops.pool_mean(V, bc, stride)
        Tk_pad = Kc.shape[2] * bc if stride == bc else Tk
        dO = grad_out.to(Q.dtype)
        delta = ops.bwd_delta(dO, O)
        dQ, dKc, dVc = ops.attention_bwd(dO, Q, Kc, Vc, LSE, delta, branch=L.BRANCH_COMPRESSED, causal=bool(causal),
                                         scale=ops.softmax_scale(D, scale), offset=Tk - Tq, dq_fp32=False, cmp_block=bc,
                                         cmp_stride=stride, cmp_offset=Tk_pad - Tq, Tk_keys=Tk)
        dK = ops.cast_from_f32(ops.pool_mean_bwd(dKc, Tk, bc, stride), K.dtype)
        dV = ops.cast_from_f32(ops.pool_mean_bwd(dVc, Tk, bc, stride), V.dtype)
        return dQ, dK, dV, None, None, None, None, None


class _SelectedFn(torch.autograd.Function):
    """Selected branch with the hand-written backward kernel."""

    @staticmethod
    def forward(ctx, Q, K, V, block_size_n, block_size_m, top_k, block_indices, causal, scale):
        if Q.dtype not in (torch.float16, torch.bfloat16):
            raise TypeError("selected branch kernels take fp16/bf16 (the reference's fp64 gradcheck route is not provided)")
        out, lse = _selected_kernel(Q, K, V, block_size_n=block_size_n, block_size_m=block_size_m, top_k=top_k,
                                    block_indices=block_indices, causal=causal, scale=scale)
        ctx.save_for_backward(Q, K, V, out, lse, block_indices)
        ctx.args = (block_size_n, block_size_m, causal, scale)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        Q, K, V, O, LSE, idx = ctx.saved_tensors
        bn, bm, causal, scale = ctx.args
        D = Q.shape[-1]
        delta = ops.bwd_delta(grad_out.to(Q.dtype), O)
        dQ, dK, dV = ops.selected_bwd(grad_out.to(Q.dtype), Q, K, V, LSE, delta, idx, bm=bm, bn=bn, causal=bool(causal),
                                      scale=ops.softmax_scale(D, scale), offset=K.shape[2] - Q.shape[2], dq_fp32=False)
        return dQ, ops.cast_from_f32(dK, K.dtype), ops.cast_from_f32(dV, V.dtype), None, None, None, None, None, None


class _SlidingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, Q, K, V, window_size, causal, scale):
        out, lse = _sliding_kernel(Q, K, V, window_size=window_size, causal=causal, scale=scale)
        ctx.save_for_backward(Q, K, V, out, lse)
        ctx.args = (window_size, causal, scale)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        Q, K, V, O, LSE = ctx.saved_tensors
        W, causal, scale = ctx.args
        D = Q.shape[-1]
        dO = grad_out.to(Q.dtype)
        delta = ops.bwd_delta(dO, O)
        dQ, dK, dV = ops.attention_bwd(dO, Q, K, V, LSE, delta, branch=L.BRANCH_SLIDING, causal=bool(causal),
                                       scale=ops.softmax_scale(D, scale), offset=K.shape[2] - Q.shape[2], dq_fp32=False,
                                       window=int(W))
        return dQ, ops.cast_from_f32(dK, K.dtype), ops.cast_from_f32(dV, V.dtype), None, None, None


class _CombineFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, out_c, out_s, out_w, gate_logits, activation):
        ctx.save_for_backward(out_c, out_s, out_w, gate_logits)
        ctx.activation = activation
        return combine(out_c, out_s, out_w, gate_logits, activation=activation)

    @staticmethod
    def backward(ctx, grad_out):
        oc, os_, ow, gl = ctx.saved_tensors
        with torch.enable_grad():
            xs = [t.detach().float().requires_grad_(True) for t in (oc, os_, ow, gl)]
            g = torch.sigmoid(xs[3]) if ctx.activation == "sigmoid" else torch.softmax(xs[3], dim=-1)
            y = g[..., 0:1] * xs[0] + g[..., 1:2] * xs[1] + g[..., 2:3] * xs[2]
            grads = torch.autograd.grad(y, xs, grad_outputs=grad_out.float())
        return tuple(gr.to(t.dtype) for gr, t in zip(grads, (oc, os_, ow, gl))) + (None,)


def _cfg(cfg, name, default):
    v = getattr(cfg, name, default)
    return default if v is None else v


def nsa_forward(Q: Tensor, K: Tensor, V: Tensor, cfg, *, gate_logits: Optional[Tensor] = None,
                block_indices: Optional[Tensor] = None, pool_proj_k: Optional[Tensor] = None,
                pool_proj_v: Optional[Tensor] = None) -> Tensor:
    """NSA combined forward.  Q [B,H,Tq,D], K/V [B,H|Hkv,Tk,D] fp16/bf16; `cfg` is any object with
    the reference's NSAConfig fields (optional extras: stride_c, force_first, force_local);
    gate_logits [B,H,Tq,3] (None = zero logits); block_indices [B,H|Hkv,nq,k] int32 (None =
    mean-pool scoring + top-k).  Returns [B,H,Tq,D] in Q's dtype on every route (the reference's
    tensor expression would promote to fp32 for fp32 gate logits, nsa/triton/gating.py:38-40; its model casts the
    logits to Q's dtype first, nsa/model/llama_nsa.py:86, so callers of the module see Q's dtype there too);
    differentiable wrt Q, K, V and gate_logits."""
    assert Q.dtype in (torch.float16, torch.bfloat16), "Q must be fp16 or bf16"
    D = Q.shape[-1]
    scale = cfg.scale if cfg.scale is not None else 1.0 / (D ** 0.5)
    learned = cfg.pool == "learned"
    if cfg.pool not in ("mean", "learned"):
        raise ValueError(f"unknown pool: {cfg.pool}")
    if learned and (pool_proj_k is None or pool_proj_v is None):
        raise ValueError("nsa_forward: pool='learned' needs pool_proj_k and pool_proj_v ([block_size_c, D], nsa/reference.py:295-296)")
    stride_c = getattr(cfg, "stride_c", None)
    ff, fl = _cfg(cfg, "force_first", 0), _cfg(cfg, "force_local", 0)
    if block_indices is None and _cfg(cfg, "scorer", "mean") == "compressed":
        from .scoring import forward_with_compressed_scorer, select_blocks_compressed
        if not (torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in (Q, K, V, gate_logits))):
            return forward_with_compressed_scorer(Q, K, V, cfg, gate_logits)
        block_indices = select_blocks_compressed(Q, K, cfg)
    elif block_indices is None:
        if _cfg(cfg, "scorer", "mean") != "mean":
            raise ValueError(f"unknown scorer: {cfg.scorer}")
        block_indices = _resolve_block_indices(Q, K, block_size_m=cfg.block_size_m, block_size_n=cfg.block_size_n,
                                               top_k=cfg.top_k, causal=cfg.causal, scale=float(scale),
                                               force_first=ff, force_local=fl,
                                               shared_per_group=bool(_cfg(cfg, "select_per_group", False)))
    needs_grad = torch.is_grad_enabled() and any(
        t is not None and t.requires_grad for t in (Q, K, V, gate_logits))
    if needs_grad and learned:
        raise NotImplementedError("nsa_forward: pool='learned' is forward-only here (no gradient kernels for the pooling weights)")
    if needs_grad:
        out_c = _CompressedFn.apply(Q, K, V, cfg.block_size_c, cfg.pool, cfg.causal, cfg.scale, stride_c)
        out_s = _SelectedFn.apply(Q, K, V, cfg.block_size_n, cfg.block_size_m, cfg.top_k, block_indices,
                                  cfg.causal, cfg.scale)
        out_w = _SlidingFn.apply(Q, K, V, cfg.window_size, cfg.causal, cfg.scale)
        if gate_logits is None:
            B, H, Tq, _ = Q.shape
            gate_logits = Q.new_full((B, H, Tq, 3), 0.0)
        out = _CombineFn.apply(out_c, out_s, out_w, gate_logits, cfg.gate_activation)
        return out if out.dtype == Q.dtype else out.to(Q.dtype)     # fp32 gate logits: same dtype as the fused route
    return _fused_forward(Q, K, V, cfg, float(scale), stride_c, gate_logits, block_indices, 1.0, 1.0, 1.0,
                          pool_proj=(pool_proj_k, pool_proj_v) if learned else None)


def _fused_forward(Q, K, V, cfg, scale, stride_c, gate_logits, block_indices, sq, sk, sv, engine=None,
                   token_major=False, pool_proj=None):
    bc = cfg.block_size_c
    stride = bc if stride_c is None else int(stride_c)
    if pool_proj is not None:
        Kc = ops.pool_learned(K, pool_proj[0], bc, stride)
        Vc = ops.pool_learned(V, pool_proj[1], bc, stride)
    else:
        Kc = ops.pool_mean(K, bc, stride, dequant_scale=sk)
        Vc = ops.pool_mean(V, bc, stride, dequant_scale=sv)
    Tq, Tk = Q.shape[2], K.shape[2]
    Tk_pad = Kc.shape[2] * bc if stride == bc else Tk
    if cfg.gate_activation not in ("sigmoid", "softmax"):
        raise ValueError(f"unknown gate_activation: {cfg.gate_activation}")
    out, _ = ops.attention_fwd(
        Q, K, V, branches=L.BRANCH_COMPRESSED | L.BRANCH_SELECTED | L.BRANCH_SLIDING, fused=True,
        causal=bool(cfg.causal), scale=scale, Kc=Kc, Vc=Vc, cmp_block=bc, cmp_stride=stride, cmp_offset=Tk_pad - Tq,
        idx=block_indices, bm=cfg.block_size_m, bn=cfg.block_size_n, window=cfg.window_size, gates=gate_logits,
        gate_act=L.GATE_SOFTMAX if cfg.gate_activation == "softmax" else L.GATE_SIGMOID,
        q_scale=sq, k_scale=sk, v_scale=sv, engine=engine, token_major=token_major)
    return out


def nsa_forward_fp8(Q: Tensor, K: Tensor, V: Tensor, scale_q: float, scale_k: float, scale_v: float, cfg, *,
                    gate_logits: Optional[Tensor] = None, block_indices: Optional[Tensor] = None) -> Tensor:
    """The combined forward on fp8 (e4m3/e5m2) Q/K/V with per-tensor scales; the operands are
    bf16(fp32(x)*scale) everywhere (Q converted as the kernel loads it, K/V once in front of it), so the
    result equals `nsa_forward` on the dequantised bf16 tensors.  Inference only.  Returns bf16."""
    assert Q.dtype in (torch.float8_e4m3fn, torch.float8_e5m2) and K.dtype == Q.dtype and V.dtype == Q.dtype
    D = Q.shape[-1]
    scale = cfg.scale if cfg.scale is not None else 1.0 / (D ** 0.5)
    if block_indices is None:
        block_indices = _resolve_block_indices(
            Q, K, block_size_m=cfg.block_size_m, block_size_n=cfg.block_size_n, top_k=cfg.top_k, causal=cfg.causal,
            scale=float(scale), force_first=_cfg(cfg, "force_first", 0), force_local=_cfg(cfg, "force_local", 0),
            q_scale=scale_q, k_scale=scale_k, shared_per_group=bool(_cfg(cfg, "select_per_group", False)))
    return _fused_forward(Q, K, V, cfg, float(scale), getattr(cfg, "stride_c", None), gate_logits, block_indices,
                          scale_q, scale_k, scale_v)


__all__ = ["nsa_forward", "nsa_forward_fp8"]
