"""Gated combination of the three branch outputs.  Same signature as the reference's
nsa/triton/gating.py:15-21; one kernel instead of six element-wise launches."""
from __future__ import annotations

from typing import Literal

from torch import Tensor

from . import ops


def combine(out_c: Tensor, out_s: Tensor, out_w: Tensor, gate_logits: Tensor,
            activation: Literal["sigmoid", "softmax"] = "sigmoid") -> Tensor:
    """g0*out_c + g1*out_s + g2*out_w with g = sigmoid / softmax of gate_logits [B,H,Tq,3]."""
    return ops.combine(out_c, out_s, out_w, gate_logits, activation)


__all__ = ["combine"]
