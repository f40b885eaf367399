"""Drop-in for the reference's `nsa.cuda` package (nsa/cuda/__init__.py:50-153): the
pre-padded, bf16, 64x64-block selected forward/backward, reached through the C launchers
with the reference's own argument lists (launch_selected_attn_fwd / _bwd)."""
from __future__ import annotations

import math
from typing import Tuple

import torch

from . import _lib as L


class _Ext:
    """Stands in for the reference's pybind module (nsa/cuda/bindings.cpp:187-215): same two
    function names, same argument order, allocates its outputs, launches on the current stream."""

    @staticmethod
    def selected_attention_fwd_cuda(Q, K, V, block_indices, block_size_m, block_size_n, top_k, offset, causal, sm_scale):
        for t in (Q, K, V, block_indices):
            if not t.is_cuda:
                raise RuntimeError("Q/K/V/block_indices must be CUDA tensors")
        if Q.dtype != torch.bfloat16 or K.dtype != torch.bfloat16 or V.dtype != torch.bfloat16:
            raise RuntimeError("Q/K/V must be bf16")
        if block_indices.dtype != torch.int32:
            raise RuntimeError("block_indices must be int32")
        if not (Q.is_contiguous() and K.is_contiguous() and V.is_contiguous() and block_indices.is_contiguous()):
            raise RuntimeError("inputs must be contiguous")
        if block_size_m != 64 or block_size_n != 64:
            raise RuntimeError("this launcher supports BLOCK_M = BLOCK_N = 64 only")
        B, H, Tq_p, D = Q.shape
        Tk_p = K.shape[2]
        if Tq_p % 64 or Tk_p % 64:
            raise RuntimeError("Tq_p / Tk_p must be multiples of 64")
        nq = Tq_p // 64
        if tuple(block_indices.shape) != (B, H, nq, top_k):
            raise RuntimeError("block_indices must be [B, H, n_q_blocks, top_k]")
        out = torch.empty_like(Q)
        lse = torch.empty((B, H, Tq_p), device=Q.device, dtype=torch.float32)
        with torch.cuda.device(Q.device):
            L.check(L.load().launch_selected_attn_fwd(
                Q.data_ptr(), K.data_ptr(), V.data_ptr(), block_indices.data_ptr(), out.data_ptr(), lse.data_ptr(),
                B * H, nq, Tq_p, Tk_p, D, top_k, int(offset), int(bool(causal)), float(sm_scale), L.stream_ptr()),
                "launch_selected_attn_fwd")
        return [out, lse]

    @staticmethod
    def selected_attention_bwd_cuda(dO, Q, K, V, LSE, Dvec, block_indices, block_size_m, block_size_n, top_k, offset,
                                    causal, sm_scale):
        if block_size_m != 64 or block_size_n != 64:
            raise RuntimeError("this launcher supports BLOCK_M = BLOCK_N = 64 only")
        for t in (dO, Q, K, V):
            if t.dtype != torch.bfloat16 or not t.is_cuda or not t.is_contiguous():
                raise RuntimeError("dO/Q/K/V must be contiguous bf16 CUDA tensors")
        B, H, Tq_p, D = Q.shape
        Tk_p = K.shape[2]
        nq = Tq_p // 64
        dQ = torch.empty_like(Q)
        dK = torch.zeros(K.shape, device=K.device, dtype=torch.float32)
        dV = torch.zeros(V.shape, device=V.device, dtype=torch.float32)
        with torch.cuda.device(Q.device):
            L.check(L.load().launch_selected_attn_bwd(
                Q.data_ptr(), K.data_ptr(), V.data_ptr(), dO.data_ptr(), LSE.contiguous().data_ptr(),
                Dvec.contiguous().data_ptr(), block_indices.contiguous().data_ptr(), dQ.data_ptr(), dK.data_ptr(),
                dV.data_ptr(), B * H, nq, Tq_p, Tk_p, D, top_k, int(offset), int(bool(causal)), float(sm_scale),
                L.stream_ptr()), "launch_selected_attn_bwd")
        return [dQ, dK, dV]


_ext = None


def _get_ext():
    global _ext
    if _ext is None:
        L.load()
        _ext = _Ext()
    return _ext


def selected_attention_cuda(Q, K, V, block_indices, block_size_n: int, block_size_m: int, top_k: int, causal: bool,
                            scale: float) -> Tuple[torch.Tensor, torch.Tensor]:
    """Pre-padded bf16 selected forward: returns (out [B,H,Tq_p,D] bf16, lse [B,H,Tq_p] fp32)."""
    assert Q.dtype == torch.bfloat16 and K.dtype == torch.bfloat16 and V.dtype == torch.bfloat16
    assert Q.is_cuda and K.is_cuda and V.is_cuda and block_indices.is_cuda
    assert block_indices.dtype == torch.int32
    assert Q.is_contiguous() and K.is_contiguous() and V.is_contiguous() and block_indices.is_contiguous()
    B, H, Tq_p, D = Q.shape
    Tk_p = K.shape[2]
    assert K.shape == V.shape == (B, H, Tk_p, D)
    assert Tq_p % block_size_m == 0 and Tk_p % block_size_n == 0
    assert block_indices.shape == (B, H, Tq_p // block_size_m, top_k)
    sm_scale = float(scale) if scale is not None else 1.0 / math.sqrt(D)
    out, lse = _get_ext().selected_attention_fwd_cuda(Q, K, V, block_indices, block_size_m, block_size_n, top_k,
                                                      Tk_p - Tq_p, bool(causal), sm_scale)
    return out, lse


def _selected_backward_cuda_native(dO, Q, K, V, O, LSE, block_indices, *, block_size_n: int, block_size_m: int,
                                   top_k: int, causal: bool, scale: float):
    """Hand-written CUDA backward through the reference-shaped launcher."""
    from . import ops
    assert Q.dtype == torch.bfloat16 and Q.is_cuda
    B, H, Tq_p, D = Q.shape
    Tk_p = K.shape[2]
    assert Tq_p % block_size_m == 0 and Tk_p % block_size_n == 0
    Dvec = ops.bwd_delta(dO, O)
    sm_scale = float(scale) if scale is not None else 1.0 / math.sqrt(D)
    dQ, dK_f, dV_f = _get_ext().selected_attention_bwd_cuda(dO, Q, K, V, LSE, Dvec, block_indices, block_size_m,
                                                            block_size_n, top_k, Tk_p - Tq_p, bool(causal), sm_scale)
    return dQ, ops.cast_from_f32(dK_f, K.dtype), ops.cast_from_f32(dV_f, V.dtype)


def selected_backward_cuda(dO, Q, K, V, O, LSE, block_indices, block_size_n: int, block_size_m: int, top_k: int,
                           causal: bool, scale: float):
    """Selected backward on pre-padded bf16 inputs (the reference dispatches this name to its
    Triton kernel because its native kernel is wrong; here the native kernel is the path)."""
    return _selected_backward_cuda_native(dO, Q, K, V, O, LSE, block_indices, block_size_n=block_size_n,
                                          block_size_m=block_size_m, top_k=top_k, causal=causal, scale=scale)


__all__ = ["selected_attention_cuda", "selected_backward_cuda"]
