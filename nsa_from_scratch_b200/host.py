"""NSA forward for HOST-resident tensors: host -> device copies, the kernels and the device -> host
copy of the result run as a three-stage pipeline over independent (batch, KV head) units.

A unit needs only its own K/V head and the query heads that share it, so unit u+1 can be on the
PCIe/NVLink-C2C bus inbound while unit u computes and unit u-1 drains outbound; the wall time of a
call tends to max(copy in, compute, copy out) instead of their sum.  Pass pinned tensors (and a pinned
`out`) for the copies to be asynchronous.
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import Tensor

from .forward import nsa_forward


def nsa_forward_host(Q: Tensor, K: Tensor, V: Tensor, cfg, *, gate_logits: Optional[Tensor] = None,
                     out: Optional[Tensor] = None, device=None) -> Tensor:
    """Q [B,H,Tq,D], K/V [B,Hkv,Tk,D], gate_logits [B,H,Tq,3] on the HOST (ideally pinned); returns the
    output [B,H,Tq,D] on the host (`out` if given, else a new pinned tensor).  Inference only."""
    if Q.is_cuda or K.is_cuda or V.is_cuda:
        raise ValueError("nsa_forward_host takes host tensors; call nsa_forward for device tensors")
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    B, H, Tq, D = Q.shape
    Hkv, Tk = K.shape[1], K.shape[2]
    G = H // Hkv
    if out is None:
        out = torch.empty((B, H, Tq, D), dtype=Q.dtype).pin_memory()
    cur = torch.cuda.current_stream(dev)
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    s_in.wait_stream(cur)
    s_out.wait_stream(cur)
    units = [(b, hk) for b in range(B) for hk in range(Hkv)]
    staged = []
    with torch.cuda.stream(s_in):
        for b, hk in units:
            hs = slice(hk * G, (hk + 1) * G)
            q = Q[b:b + 1, hs].to(dev, non_blocking=True)
            k = K[b:b + 1, hk:hk + 1].to(dev, non_blocking=True)
            v = V[b:b + 1, hk:hk + 1].to(dev, non_blocking=True)
            g = gate_logits[b:b + 1, hs].to(dev, non_blocking=True) if gate_logits is not None else None
            ev = torch.cuda.Event()
            ev.record(s_in)
            staged.append((q, k, v, g, ev))
    done = []
    for (b, hk), (q, k, v, g, ev) in zip(units, staged):
        cur.wait_event(ev)
        for t in (q, k, v, g):
            if t is not None:
                t.record_stream(cur)
        o = nsa_forward(q, k, v, cfg, gate_logits=g)
        ev2 = torch.cuda.Event()
        ev2.record(cur)
        done.append((b, hk, o, ev2))
    with torch.cuda.stream(s_out):
        for b, hk, o, ev2 in done:
            s_out.wait_event(ev2)
            o.record_stream(s_out)
            out[b:b + 1, hk * G:(hk + 1) * G].copy_(o, non_blocking=True)
    cur.wait_stream(s_out)
    return out


__all__ = ["nsa_forward_host"]
