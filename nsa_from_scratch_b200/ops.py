"""Tensor-level wrappers over the C ABI: check tensors, allocate outputs, pass raw pointers.

torch is used only for device memory, dtypes and the current stream.  Nothing here computes
on the host and nothing falls back to torch arithmetic.
"""
from __future__ import annotations

import ctypes as C
import math
from typing import Optional, Tuple

import torch
from torch import Tensor

from . import _lib as L

_ENGINE = L.ENGINE_AUTO


def set_engine(name: str) -> None:
    """Which attention-forward kernel nsa_attention_fwd uses: "auto" (tcgen05 when the shape
    qualifies, else generic), "generic" or "tcgen05" (error when the shape does not qualify)."""
    global _ENGINE
    _ENGINE = {"auto": L.ENGINE_AUTO, "generic": L.ENGINE_GENERIC, "tcgen05": L.ENGINE_TCGEN05}[name]


def engine() -> int:
    return _ENGINE


_BWD_ENGINE = L.ENGINE_AUTO


def set_bwd_engine(name: str) -> None:
    """Which engine nsa_attention_bwd uses: "auto" (tcgen05 for the selected branch when the shape qualifies,
    else generic), "generic" (mma.sync with fp32 atomic adds) or "tcgen05" (error when the shape does not qualify)."""
    global _BWD_ENGINE
    _BWD_ENGINE = {"auto": L.ENGINE_AUTO, "generic": L.ENGINE_GENERIC, "tcgen05": L.ENGINE_TCGEN05}[name]


def device_status() -> None:
    """Synchronise the current stream and raise if a kernel gave up on a bounded device-side wait."""
    L.check(L.load().nsa_device_status(L.stream_ptr()), "nsa_device_status")


_STRICT_LAYOUT = False
_warned_layout = set()


def set_strict_layout(flag: bool) -> None:
    """The kernels read dense row-major tensors.  The reference's wrappers call .contiguous() on whatever they are
    given (nsa/triton/selected.py:239-241, compressed.py:243-245), which copies a strided operand in full; so do these
    wrappers by default, with one warning per operand name, because such a copy on the hot path is rarely intended.
    set_strict_layout(True) turns it into an error."""
    global _STRICT_LAYOUT
    _STRICT_LAYOUT = bool(flag)


def _dense(t: Tensor, name: str) -> Tensor:
    if t.is_contiguous():
        return t
    if _STRICT_LAYOUT:
        raise ValueError(f"{name} is not contiguous (shape {tuple(t.shape)}, strides {t.stride()}); the kernels take dense "
                         "row-major tensors and strict layout checking is on")
    if name not in _warned_layout:
        _warned_layout.add(name)
        import warnings
        warnings.warn(f"nsa_from_scratch_b200: {name} is not contiguous and is being copied ({t.numel() * t.element_size()} bytes) "
                      "before the launch; pass a dense tensor, or ops.set_strict_layout(True) to make this an error", stacklevel=3)
    return t.contiguous()


_16 = (torch.float16, torch.bfloat16)
_8 = (torch.float8_e4m3fn, torch.float8_e5m2)


def _need_cuda(*ts: Tensor) -> None:
    for t in ts:
        if t is not None and not t.is_cuda:
            raise RuntimeError("nsa_from_scratch_b200 kernels need CUDA tensors (there is no CPU path)")


def softmax_scale(D: int, scale: Optional[float]) -> float:
    return float(scale) if scale is not None else 1.0 / math.sqrt(D)


def n_pooled(T: int, block: int, stride: Optional[int] = None) -> int:
    stride = block if stride is None else stride
    if stride == block:
        return (T + block - 1) // block
    return (T - block) // stride + 1 if T >= block else 0


def pool_mean(x: Tensor, block: int, stride: Optional[int] = None, dequant_scale: float = 1.0) -> Tensor:
    """[B,H,T,D] -> [B,H,n,D] window means (16-bit in -> same type; fp8 in -> bf16)."""
    _need_cuda(x)
    B, H, T, D = x.shape
    stride = block if stride is None else stride
    n = n_pooled(T, block, stride)
    x = _dense(x, "x")
    out = torch.empty((B, H, n, D), device=x.device, dtype=torch.bfloat16 if x.dtype in _8 else x.dtype)
    with torch.cuda.device(x.device):
        L.check(L.load().nsa_pool_mean(x.data_ptr(), out.data_ptr(), B, H, T, D, block, stride, n,
                                       L.dtype_code(x.dtype), float(dequant_scale), L.stream_ptr()), "nsa_pool_mean")
    return out


def pool_learned(x: Tensor, w: Tensor, block: int, stride: Optional[int] = None) -> Tensor:
    """[B,H,T,D] 16-bit, w [block, D] -> [B,H,n,D]: window c is sum_s x[c*stride+s] * w[s] (fp32 sum, one rounding)."""
    _need_cuda(x, w)
    B, H, T, D = x.shape
    stride = block if stride is None else stride
    if w.shape != (block, D):
        raise ValueError(f"pool_learned: weights must be [{block}, {D}], got {tuple(w.shape)}")
    n = n_pooled(T, block, stride)
    x = _dense(x, "x")
    w = w.detach().to(torch.float32).contiguous()
    out = torch.empty((B, H, n, D), device=x.device, dtype=x.dtype)
    with torch.cuda.device(x.device):
        L.check(L.load().nsa_pool_learned(x.data_ptr(), w.data_ptr(), out.data_ptr(), B, H, T, D, block, stride, n,
                                          L.dtype_code(x.dtype), L.stream_ptr()), "nsa_pool_learned")
    return out


def select_blocks_from_means(Qb: Tensor, Kb: Tensor, *, top_k: int, bm: int, bn: int, offset: int, causal: bool,
                             scale: float, force_first: int = 0, force_local: int = 0,
                             shared_per_group: bool = False) -> Tensor:
    _need_cuda(Qb, Kb)
    B, H, nq, D = Qb.shape
    Hkv, nk = Kb.shape[1], Kb.shape[2]
    k_out = min(top_k, nk)
    idx = torch.empty((B, Hkv if shared_per_group else H, nq, k_out), device=Qb.device, dtype=torch.int32)
    with torch.cuda.device(Qb.device):
        L.check(L.load().nsa_select_blocks(Qb.data_ptr(), Kb.data_ptr(), idx.data_ptr(), B, H, Hkv, nq, nk, D, top_k,
                                           bm, bn, offset, int(causal), float(scale), force_first, force_local,
                                           int(shared_per_group), L.dtype_code(Qb.dtype), L.stream_ptr()), "nsa_select_blocks")
    return idx


def cmp_block_scores(Q: Tensor, Kc: Tensor, lse: Tensor, *, nk: int, cmp_block: int, cmp_stride: int, cmp_offset: int,
                     bn: int, sel_offset: int, causal: bool, scale: float, force_first: int = 0, force_local: int = 0,
                     shared_per_group: bool = False) -> Tensor:
    """fp32 [B,H|Hkv,nq,nk] selection scores from the compressed branch's probabilities (lse = its log-sum-exp)."""
    _need_cuda(Q, Kc, lse)
    B, H, Tq, D = Q.shape
    Hkv, Nc = Kc.shape[1], Kc.shape[2]
    Q, Kc, lse = _dense(Q, "Q"), _dense(Kc, "Kc"), lse.float().contiguous()
    if Kc.dtype != Q.dtype or Q.dtype not in _16:
        raise TypeError("cmp_block_scores: Q and the pooled K must share a 16-bit dtype")
    nq = (Tq + 63) // 64
    scores = torch.empty((B, Hkv if shared_per_group else H, nq, nk), device=Q.device, dtype=torch.float32)
    # tcgen05 kernel where it applies: D in {64,128} and the four score rows of a work item fit shared memory
    fixed = 4 * (D // 64) * 128 * 128 + (256 + 1024 + 4 * nk) * 4 + 1024
    if (_ENGINE != L.ENGINE_GENERIC and D in (64, 128) and (bn + cmp_block) // cmp_stride + 1 <= 64 and fixed <= 225 * 1024
            and bn % cmp_stride == 0 and cmp_block % cmp_stride == 0):
        scratch = torch.empty((B, H, nq, nk), device=Q.device, dtype=torch.float32)
        with torch.cuda.device(Q.device):
            L.check(L.load().nsa_cmp_block_scores_tc(Q.data_ptr(), Kc.data_ptr(), lse.data_ptr(), scores.data_ptr(), scratch.data_ptr(),
                                                     B, H, Hkv, Tq, Nc, D, nk, cmp_block, cmp_stride, cmp_offset, bn, sel_offset,
                                                     int(causal), float(scale), force_first, force_local, int(shared_per_group),
                                                     L.dtype_code(Q.dtype), L.stream_ptr()), "nsa_cmp_block_scores_tc")
        return scores
    with torch.cuda.device(Q.device):
        L.check(L.load().nsa_cmp_block_scores(Q.data_ptr(), Kc.data_ptr(), lse.data_ptr(), scores.data_ptr(), B, H, Hkv, Tq, Nc, D,
                                              nk, cmp_block, cmp_stride, cmp_offset, bn, sel_offset, int(causal), float(scale),
                                              force_first, force_local, int(shared_per_group), L.dtype_code(Q.dtype),
                                              L.stream_ptr()), "nsa_cmp_block_scores")
    return scores


def topk_from_scores(scores: Tensor, *, top_k: int, bm: int, bn: int, offset: int, causal: bool) -> Tensor:
    _need_cuda(scores)
    B, H, nq, nk = scores.shape
    scores = scores.float().contiguous()
    idx = torch.empty((B, H, nq, min(top_k, nk)), device=scores.device, dtype=torch.int32)
    with torch.cuda.device(scores.device):
        L.check(L.load().nsa_topk_from_scores(scores.data_ptr(), idx.data_ptr(), B * H, nq, nk, top_k, bm, bn, offset,
                                              int(causal), L.stream_ptr()), "nsa_topk_from_scores")
    return idx


def attention_fwd(
    Q: Tensor, K: Tensor, V: Tensor, *, branches: int, fused: bool, causal: bool, scale: float,
    Kc: Optional[Tensor] = None, Vc: Optional[Tensor] = None, cmp_block: int = 0, cmp_stride: int = 0,
    cmp_offset: int = 0, idx: Optional[Tensor] = None, bm: int = 64, bn: int = 64, window: int = 0,
    gates: Optional[Tensor] = None, gate_act: int = L.GATE_SIGMOID, offset: Optional[int] = None,
    q_scale: float = 1.0, k_scale: float = 1.0, v_scale: float = 1.0, engine: Optional[int] = None,
    want_lse: bool = True, token_major: bool = False, nsplit: int = 1, dyn_len: Optional[Tensor] = None,
    accumulate_into: Optional[Tensor] = None, fused_lse: bool = False, dequant_kv: Optional[bool] = None,
) -> Tuple[Tensor, Optional[Tensor]]:
    """One launch of nsa_attention_fwd.  Returns (out, lse); lse is None for fused launches.
    `token_major`: gates are [B,Tq,H,3] and the result comes back as [B,Tq,H,D] (Q, K, V stay
    [B,H,T,D]) -- the layouts on either side of the call in the reference's attention module.
    `nsplit` > 1 (fused launches): each work item's key tiles are spread over that many thread blocks, for
    launches with few query blocks and long key ranges (decoding).  `dyn_len`: int32 device scalar with the
    number of filled key positions; K/V/Kc/Vc are then allocations and every offset is derived on the device.
    `accumulate_into`: the output of an earlier fused launch (other branches); this launch adds its branches to it
    and returns the same tensor.  `fused_lse`: a fused launch of ONE branch also returns that branch's lse.
    `dequant_kv` (fp8 inputs): True/False forces / forbids the one-off dequantisation of K and V in front of the
    launch; None decides by kernel (see below).  The results are identical either way."""
    _need_cuda(Q, K, V)
    B, H, Tq, D = Q.shape
    Hkv, Tk = K.shape[1], K.shape[2]
    if K.shape != (B, Hkv, Tk, D) or V.shape != K.shape:
        raise ValueError(f"K/V shapes {tuple(K.shape)}/{tuple(V.shape)} do not match Q {tuple(Q.shape)}")
    if H % Hkv:
        raise ValueError(f"query heads {H} not a multiple of KV heads {Hkv}")
    if V.dtype != K.dtype or (K.dtype != Q.dtype and not (Q.dtype in _8 and K.dtype == torch.bfloat16)):
        raise TypeError("Q, K, V must share a dtype (or bf16 K/V beside an fp8 Q)")
    Q, K, V = _dense(Q, "Q"), _dense(K, "K"), _dense(V, "V")
    eng = _ENGINE if engine is None else engine
    if Q.dtype in _8 and K.dtype == Q.dtype and eng != L.ENGINE_GENERIC and D in (64, 128):
        # The tcgen05 kernel takes an fp8 Q with bf16 K/V: a K/V tile is used by every query block that attends it,
        # so K and V are dequantised ONCE here (with GQA they are a small fraction of Q) instead of once per use
        # inside the kernel, where the conversion, not the tensor pipe, set the pace; Q's tiles are used once and
        # stay fp8 in HBM.  A selected-only launch with one list per head at D=64 runs on the generic kernel.
        per_head_sel = (not fused and branches == L.BRANCH_SELECTED and idx is not None and idx.shape[1] == H and D == 64
                        and eng == L.ENGINE_AUTO)
        if (not per_head_sel) if dequant_kv is None else dequant_kv:
            K, V = fp8_dequantize(K, k_scale), fp8_dequantize(V, v_scale)
    out_dtype = torch.bfloat16 if Q.dtype in _8 else Q.dtype
    if accumulate_into is not None:
        out = accumulate_into
        if not fused or out.shape != ((B, Tq, H, D) if token_major else (B, H, Tq, D)) or out.dtype != out_dtype or not out.is_contiguous():
            raise ValueError("accumulate_into must be the contiguous output of a fused launch of the same problem")
    else:
        out = torch.empty((B, Tq, H, D) if token_major else (B, H, Tq, D), device=Q.device, dtype=out_dtype)
    lse = torch.empty((B, H, Tq), device=Q.device, dtype=torch.float32) if ((want_lse and not fused) or (fused and fused_lse)) else None
    a = L.FwdArgs()
    a.accumulate = int(accumulate_into is not None)
    a.io_layout = (L.IO_OUT_BTHD | L.IO_GATES_BTHD) if token_major else 0
    a.Q, a.K, a.V, a.out, a.lse = Q.data_ptr(), K.data_ptr(), V.data_ptr(), out.data_ptr(), L.ptr(lse)
    a.B, a.H, a.Hkv, a.Tq, a.Tk, a.D = B, H, Hkv, Tq, Tk, D
    a.offset = Tk - Tq if offset is None else offset
    a.causal, a.branches, a.fused, a.gate_act = int(causal), branches, int(fused), gate_act
    a.q_dtype, a.kv_dtype = L.dtype_code(Q.dtype), L.dtype_code(K.dtype)
    a.scale, a.q_scale, a.k_scale, a.v_scale = float(scale), float(q_scale), float(k_scale), float(v_scale)
    a.engine = eng
    keep = [Q, K, V]
    if branches & L.BRANCH_COMPRESSED:
        Kc, Vc = _dense(Kc, "Kc"), _dense(Vc, "Vc")
        keep += [Kc, Vc]
        a.Kc, a.Vc, a.Nc = Kc.data_ptr(), Vc.data_ptr(), Kc.shape[2]
        a.cmp_block, a.cmp_stride, a.cmp_offset = cmp_block, cmp_stride, cmp_offset
    if branches & L.BRANCH_SELECTED:
        idx = idx.to(torch.int32).contiguous()
        keep.append(idx)
        nq = (Tq + bm - 1) // bm
        if idx.dim() != 4 or idx.shape[0] != B or idx.shape[1] not in (H, Hkv) or idx.shape[2] != nq:
            raise ValueError(f"block_indices shape {tuple(idx.shape)} does not match (B={B}, H={H}|{Hkv}, nq={nq}, k)")
        a.idx, a.Hi, a.nq, a.top_k, a.bm, a.bn = idx.data_ptr(), idx.shape[1], nq, idx.shape[3], bm, bn
        a.sel_key_limit = ((Tk + bn - 1) // bn) * bn
    if branches & L.BRANCH_SLIDING:
        a.window = int(window)
    if fused and gates is not None:
        gates = _dense(gates, "gates")
        keep.append(gates)
        want = (B, Tq, H, 3) if token_major else (B, H, Tq, 3)
        if gates.shape != want:
            raise ValueError(f"gate_logits shape {tuple(gates.shape)} != {want}")
        a.gates, a.gate_dtype = gates.data_ptr(), L.dtype_code(gates.dtype)
    if fused and (nsplit > 1 or dyn_len is not None) and Q.dtype in _16:
        nsplit = max(1, int(nsplit))
        scratch = torch.empty((B * H * Tq * nsplit * 3 * (D + 4),), device=Q.device, dtype=torch.float32)
        keep.append(scratch)
        a.nsplit, a.split_scratch, a.split_scratch_bytes = nsplit, scratch.data_ptr(), scratch.numel() * 4
    if dyn_len is not None:
        if dyn_len.dtype != torch.int32 or not dyn_len.is_cuda or dyn_len.numel() != 1:
            raise ValueError("dyn_len must be a one-element int32 CUDA tensor")
        keep.append(dyn_len)
        a.dyn_len = dyn_len.data_ptr()
    with torch.cuda.device(Q.device):
        L.check(L.load().nsa_attention_fwd(C.byref(a), L.stream_ptr()), "nsa_attention_fwd")
    return out, lse


def bwd_delta(dO: Tensor, O: Tensor) -> Tensor:
    _need_cuda(dO, O)
    dO, O = _dense(dO, "dO"), _dense(O, "O")
    D = dO.shape[-1]
    delta = torch.empty(dO.shape[:-1], device=dO.device, dtype=torch.float32)
    with torch.cuda.device(dO.device):
        L.check(L.load().nsa_bwd_delta(dO.data_ptr(), O.data_ptr(), delta.data_ptr(), delta.numel(), D,
                                       L.dtype_code(dO.dtype), L.stream_ptr()), "nsa_bwd_delta")
    return delta


def attention_bwd(dO: Tensor, Q: Tensor, K: Tensor, V: Tensor, lse: Tensor, delta: Tensor, *, branch: int, causal: bool,
                  scale: float, offset: int, dq_fp32: bool, idx: Optional[Tensor] = None, bm: int = 64, bn: int = 64,
                  window: int = 0, cmp_block: int = 0, cmp_stride: int = 0, cmp_offset: int = 0,
                  Tk_keys: Optional[int] = None) -> Tuple[Tensor, Tensor, Tensor]:
    """Backward of one branch.  For the compressed branch K/V are the POOLED tensors [B,Hkv,Nc,D] and the
    returned dK/dV are their fp32 gradients (Tk_keys = length of the raw key sequence).  Returns
    (dQ in Q.dtype or fp32, dK fp32, dV fp32)."""
    _need_cuda(dO, Q, K, V, lse, delta)
    B, H, Tq, D = Q.shape
    Hkv, rows = K.shape[1], K.shape[2]
    dO, Q, K, V = _dense(dO, "dO"), _dense(Q, "Q"), _dense(K, "K"), _dense(V, "V")
    lse, delta = _dense(lse, "lse"), _dense(delta, "delta")
    dQ = torch.empty((B, H, Tq, D), device=Q.device, dtype=torch.float32 if dq_fp32 else Q.dtype)
    dK = torch.zeros((B, Hkv, rows, D), device=Q.device, dtype=torch.float32)
    dV = torch.zeros((B, Hkv, rows, D), device=Q.device, dtype=torch.float32)
    a = L.BwdArgs()
    a.Q, a.K, a.V, a.dO = Q.data_ptr(), K.data_ptr(), V.data_ptr(), dO.data_ptr()
    a.lse, a.delta = lse.data_ptr(), delta.data_ptr()
    a.dQ, a.dK_f, a.dV_f = dQ.data_ptr(), dK.data_ptr(), dV.data_ptr()
    a.B, a.H, a.Hkv, a.Tq, a.D = B, H, Hkv, Tq, D
    a.Tk = rows if Tk_keys is None else Tk_keys
    a.branch, a.offset, a.causal, a.dtype = branch, offset, int(causal), L.dtype_code(Q.dtype)
    a.dq_dtype = L.FP32 if dq_fp32 else a.dtype
    a.scale = float(scale)
    if branch == L.BRANCH_SELECTED:
        idx = idx.to(torch.int32).contiguous()
        a.idx, a.Hi, a.nq, a.top_k, a.bm, a.bn = idx.data_ptr(), idx.shape[1], (Tq + bm - 1) // bm, idx.shape[3], bm, bn
        a.sel_key_limit = ((rows + bn - 1) // bn) * bn
    elif branch == L.BRANCH_SLIDING:
        a.window = int(window)
    else:
        a.Nc, a.cmp_block, a.cmp_stride, a.cmp_offset = rows, cmp_block, cmp_stride, cmp_offset
    a.engine = _BWD_ENGINE
    with torch.cuda.device(Q.device):
        lib = L.load()
        scratch = None
        if _BWD_ENGINE != L.ENGINE_GENERIC:
            need = int(lib.nsa_attention_bwd_scratch_bytes(C.byref(a)))
            if need > 0:      # the tcgen05 engine takes this shape: give it its scratch (inverted lists, partial sums)
                scratch = torch.empty(need, device=Q.device, dtype=torch.uint8)
                a.scratch, a.scratch_bytes = scratch.data_ptr(), need
        L.check(lib.nsa_attention_bwd(C.byref(a), L.stream_ptr()), "nsa_attention_bwd")
    return dQ, dK, dV


def selected_bwd(dO: Tensor, Q: Tensor, K: Tensor, V: Tensor, lse: Tensor, delta: Tensor, idx: Tensor, *, bm: int,
                 bn: int, causal: bool, scale: float, offset: int, dq_fp32: bool) -> Tuple[Tensor, Tensor, Tensor]:
    """Returns (dQ in Q.dtype or fp32, dK fp32, dV fp32)."""
    return attention_bwd(dO, Q, K, V, lse, delta, branch=L.BRANCH_SELECTED, causal=causal, scale=scale, offset=offset,
                         dq_fp32=dq_fp32, idx=idx, bm=bm, bn=bn)


def pool_mean_bwd(dxc: Tensor, T: int, block: int, stride: int) -> Tensor:
    """fp32 [B,H,n,D] gradients of pooled rows -> fp32 [B,H,T,D] gradients of the rows."""
    _need_cuda(dxc)
    B, H, n, D = dxc.shape
    dxc = _dense(dxc, "dxc")
    dx = torch.zeros((B, H, T, D), device=dxc.device, dtype=torch.float32)
    with torch.cuda.device(dxc.device):
        L.check(L.load().nsa_pool_mean_bwd(dxc.data_ptr(), dx.data_ptr(), B, H, T, D, block, stride, n, L.stream_ptr()),
                "nsa_pool_mean_bwd")
    return dx


def cast_from_f32(x: Tensor, dtype: torch.dtype) -> Tensor:
    _need_cuda(x)
    x = _dense(x, "x")
    out = torch.empty(x.shape, device=x.device, dtype=dtype)
    with torch.cuda.device(x.device):
        L.check(L.load().nsa_cast_from_f32(x.data_ptr(), out.data_ptr(), x.numel(), L.dtype_code(dtype), L.stream_ptr()),
                "nsa_cast_from_f32")
    return out


def rope_to_heads(x: Tensor, cos: Optional[Tensor], sin: Optional[Tensor], dtype: torch.dtype = torch.bfloat16) -> Tensor:
    """x [B,T,H,D] (fp32/bf16/fp16) -> rope(x) as [B,H,T,D] in `dtype`, one pass; cos/sin [T,D] or None (no rotation)."""
    _need_cuda(x)
    if x.dim() != 4:
        raise ValueError(f"rope_to_heads: x must be [B,T,H,D], got {tuple(x.shape)}")
    B, T, H, D = x.shape
    x = _dense(x, "x")
    if (cos is None) != (sin is None):
        raise ValueError("rope_to_heads: give both cos and sin or neither")
    cs_code = 0
    if cos is not None:
        _need_cuda(cos, sin)
        if cos.shape != (T, D) or sin.shape != (T, D) or cos.dtype != sin.dtype:
            raise ValueError(f"rope_to_heads: cos/sin must be [{T},{D}] of one dtype, got {tuple(cos.shape)}/{tuple(sin.shape)}")
        cos, sin = _dense(cos, "cos"), _dense(sin, "sin")
        cs_code = L.dtype_code(cos.dtype)
    y = torch.empty((B, H, T, D), device=x.device, dtype=dtype)
    with torch.cuda.device(x.device):
        L.check(L.load().nsa_rope_to_heads(x.data_ptr(), y.data_ptr(), L.ptr(cos), L.ptr(sin), B, T, H, D,
                                           L.dtype_code(x.dtype), cs_code, L.dtype_code(dtype), L.stream_ptr()),
                "nsa_rope_to_heads")
    return y


def copy_rows(dst: Tensor, src: Tensor) -> None:
    """dst[r] = src[r] for [R, ...] views whose trailing dimensions are dense and whose rows are a fixed
    stride apart; exactly one side on the device, the other on the host (pinned for an asynchronous
    copy).  One strided DMA on the current stream of the device tensor's device."""
    if dst.shape != src.shape or dst.dtype != src.dtype or dst.dim() < 2:
        raise ValueError("copy_rows: dst and src must be [R, ...] views of equal shape and dtype")
    if dst.is_cuda == src.is_cuda:
        raise ValueError("copy_rows: exactly one of dst / src must be a CUDA tensor")
    for t in (dst, src):
        if not t[0].is_contiguous():
            raise ValueError("copy_rows: the trailing dimensions must be dense")
    isz = dst.element_size()
    row_bytes = dst[0].numel() * isz
    rows = dst.shape[0]
    dp = (dst.stride(0) if rows > 1 else dst[0].numel()) * isz
    sp = (src.stride(0) if rows > 1 else src[0].numel()) * isz
    dev = dst.device if dst.is_cuda else src.device
    with torch.cuda.device(dev):
        L.check(L.load().nsa_memcpy_2d(dst.data_ptr(), dp, src.data_ptr(), sp, row_bytes, rows, 1 if dst.is_cuda else 0,
                                       L.stream_ptr()), "nsa_memcpy_2d")


def combine(out_c: Tensor, out_s: Tensor, out_w: Tensor, gate_logits: Tensor, activation: str) -> Tensor:
    _need_cuda(out_c, out_s, out_w, gate_logits)
    if activation not in ("sigmoid", "softmax"):
        raise ValueError(f"unknown activation: {activation}")
    if out_c.dtype not in _16 or out_s.dtype != out_c.dtype or out_w.dtype != out_c.dtype:
        raise TypeError("combine: branch outputs must share a 16-bit dtype")
    if gate_logits.dtype not in (out_c.dtype, torch.float32):
        raise TypeError("combine: gate logits must have the branch dtype or fp32")
    B, H, Tq, D = out_c.shape
    if gate_logits.shape != (B, H, Tq, 3):
        raise ValueError(f"gate_logits shape {tuple(gate_logits.shape)} != {(B, H, Tq, 3)}")
    out_c, out_s, out_w, g = _dense(out_c, "out_c"), _dense(out_s, "out_s"), _dense(out_w, "out_w"), _dense(gate_logits, "gate_logits")
    out = torch.empty((B, H, Tq, D), device=out_c.device, dtype=torch.float32 if g.dtype == torch.float32 else out_c.dtype)
    with torch.cuda.device(out_c.device):
        L.check(L.load().nsa_combine(out_c.data_ptr(), out_s.data_ptr(), out_w.data_ptr(), g.data_ptr(), out.data_ptr(),
                                     B * H * Tq, D, L.GATE_SOFTMAX if activation == "softmax" else L.GATE_SIGMOID,
                                     L.dtype_code(out_c.dtype), L.dtype_code(g.dtype), L.stream_ptr()), "nsa_combine")
    return out


def fp8_absmax(x: Tensor) -> Tensor:
    _need_cuda(x)
    x = _dense(x, "x")
    out = torch.zeros(1, device=x.device, dtype=torch.float32)
    with torch.cuda.device(x.device):
        L.check(L.load().nsa_fp8_absmax(x.data_ptr(), x.numel(), L.dtype_code(x.dtype), out.data_ptr(), L.stream_ptr()),
                "nsa_fp8_absmax")
    return out


def fp8_dequantize(x8: Tensor, scale: float) -> Tensor:
    """bf16(fp32(x8) * scale): the tensor the reference's wrapper attends on (nsa/triton/fp8.py:67-69)."""
    _need_cuda(x8)
    x8 = _dense(x8, "x8")
    out = torch.empty(x8.shape, device=x8.device, dtype=torch.bfloat16)
    with torch.cuda.device(x8.device):
        L.check(L.load().nsa_fp8_dequantize(x8.data_ptr(), out.data_ptr(), x8.numel(), L.dtype_code(x8.dtype), float(scale),
                                            L.stream_ptr()), "nsa_fp8_dequantize")
    return out


def fp8_quantize(x: Tensor, fmt: torch.dtype, scale: float) -> Tensor:
    _need_cuda(x)
    x = _dense(x, "x")
    out = torch.empty(x.shape, device=x.device, dtype=torch.uint8)
    with torch.cuda.device(x.device):
        L.check(L.load().nsa_fp8_quantize(x.data_ptr(), out.data_ptr(), x.numel(), L.dtype_code(x.dtype),
                                          L.dtype_code(fmt), float(scale), L.stream_ptr()), "nsa_fp8_quantize")
    return out.view(fmt)
