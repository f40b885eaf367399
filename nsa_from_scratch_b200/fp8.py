"""FP8 storage path.  Same signatures as the reference's nsa/triton/fp8.py:20-58; the
dequantisation bf16(fp32(x)*scale) of Q happens inside the attention kernel while its tiles
are staged; K and V, whose tiles every attending query block uses again, are dequantised once
in front of the tcgen05 kernel (ops.attention_fwd) and inside the generic kernel otherwise."""
from __future__ import annotations

from typing import Optional

import torch

from . import _lib as L
from . import ops

_E4M3_MAX = 448.0
_E5M2_MAX = 57344.0


def quantize_to_fp8(x: torch.Tensor, *, fmt: torch.dtype = torch.float8_e4m3fn, eps: float = 1e-12
                    ) -> tuple[torch.Tensor, float]:
    """Per-tensor absmax quantisation: returns (x_fp8, scale) with x ~= x_fp8 * scale."""
    if fmt == torch.float8_e4m3fn:
        fmt_max = _E4M3_MAX
    elif fmt == torch.float8_e5m2:
        fmt_max = _E5M2_MAX
    else:
        raise ValueError(f"unsupported fp8 format: {fmt}")
    absmax = max(float(ops.fp8_absmax(x.detach()).item()), eps)
    scale = absmax / fmt_max
    return ops.fp8_quantize(x.detach(), fmt, scale), scale


def selected_attention_fp8(
    Q: torch.Tensor, K: torch.Tensor, V: torch.Tensor, scale_q: float, scale_k: float, scale_v: float, *,
    block_size_n: int = 64, block_size_m: int = 64, top_k: int = 16, block_scores: Optional[torch.Tensor] = None,
    block_indices: Optional[torch.Tensor] = None, causal: bool = True, scale: Optional[float] = None,
) -> tuple[torch.Tensor, torch.Tensor]:
    """Selected branch on fp8 Q/K/V; compute is bf16.  Returns (out bf16, lse fp32)."""
    assert Q.dtype in (torch.float8_e4m3fn, torch.float8_e5m2), f"Q must be fp8; got {Q.dtype}"
    assert K.dtype == Q.dtype and V.dtype == Q.dtype
    B, H, Tq, D = Q.shape
    Tk = K.shape[2]
    nq = (Tq + block_size_m - 1) // block_size_m
    nk = (Tk + block_size_n - 1) // block_size_n
    if block_indices is None:
        assert block_scores is not None, "selected_attention_fp8 requires either block_scores or block_indices"
        assert block_scores.shape == (B, H, nq, nk)
        block_indices = ops.topk_from_scores(block_scores.float(), top_k=top_k, bm=block_size_m, bn=block_size_n,
                                             offset=Tk - Tq, causal=bool(causal))
    return ops.attention_fwd(Q, K, V, branches=L.BRANCH_SELECTED, fused=False, causal=bool(causal),
                             scale=ops.softmax_scale(D, scale), idx=block_indices, bm=block_size_m, bn=block_size_n,
                             q_scale=scale_q, k_scale=scale_k, v_scale=scale_v)


__all__ = ["selected_attention_fp8", "quantize_to_fp8"]
