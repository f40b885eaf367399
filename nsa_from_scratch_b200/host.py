"""NSA forward for HOST-resident tensors: host -> device copies, the kernels and the device -> host
copy of the result run as a three-stage pipeline over independent units.

A unit is (batch, KV head, query chunk).  It needs the query heads that share the KV head, for its
own chunk of positions only, and -- causal attention -- the keys up to the chunk's end, of which all
but the newest chunk are on the device already.  So unit u+1 is on the PCIe / C2C link inbound while
unit u computes and unit u-1 drains outbound, the wall time of a call tends to max(copy in, compute,
copy out), and what the pipeline cannot hide (the first copy in, the last compute and copy out) shrinks
with the chunk.  Pass pinned tensors (and a pinned `out`) for the copies to be asynchronous.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
from torch import Tensor

from . import ops
from .forward import nsa_forward


def _chunk_rows(cfg, Tq: int, Tk: int, want: Optional[int]) -> int:
    """Query rows per unit.  Chunking keeps every row's arithmetic identical only when all block
    grids (compression, selection keys, selection queries, the kernels' 64-row tiles) line up at
    each chunk boundary and the lengths carry no ragged tail; otherwise one chunk = the whole call."""
    if not want or want >= Tq or not cfg.causal or Tk < Tq:
        return Tq
    m = math.lcm(64, int(cfg.block_size_c), int(cfg.block_size_n), int(cfg.block_size_m))
    stride_c = getattr(cfg, "stride_c", None)
    if stride_c:
        m = math.lcm(m, int(stride_c))
    if Tq % m or Tk % m:
        return Tq
    return max(m, want // m * m)


_streams = {}


def _side_streams(dev):
    """One copy-in and one copy-out stream per device, created once."""
    key = (dev.type, dev.index if dev.index is not None else torch.cuda.current_device())
    if key not in _streams:
        _streams[key] = (torch.cuda.Stream(dev), torch.cuda.Stream(dev))
    return _streams[key]


def nsa_forward_host(Q: Tensor, K: Tensor, V: Tensor, cfg, *, gate_logits: Optional[Tensor] = None,
                     out: Optional[Tensor] = None, device=None, chunk_rows: Optional[int] = 16384,
                     non_blocking: bool = False, block_indices_fn=None):
    """Q [B,H,Tq,D], K/V [B,Hkv,Tk,D], gate_logits [B,H,Tq,3] on the HOST (ideally pinned); returns the
    output [B,H,Tq,D] on the host (`out` if given, else a new pinned tensor).  Inference only.
    The call returns when the last device -> host copy has landed, so the result can be read on the CPU at once.
    With non_blocking=True it returns (out, event) as soon as everything is queued; the caller must
    event.synchronize() (or synchronize the device) before reading `out`.
    `block_indices_fn(q_dev, k_dev)`: where the block lists of a unit come from instead of nsa_forward's own
    selection -- a rank that holds only some query heads of a KV head passes the selection that all-gathers the
    heads' block means (parallel.resolve_block_indices_split).
    `chunk_rows`: query positions per pipeline unit (None = whole sequences).  Smaller chunks shorten the
    unhidden head and tail of the pipeline but cost a fixed host-side launch sequence each; 16384 was the
    fastest at 64k tokens x 64 heads on a B200 over PCIe (29.9 ms; 8192: 31.7, whole sequences: 32.3)."""
    if Q.is_cuda or K.is_cuda or V.is_cuda:
        raise ValueError("nsa_forward_host takes host tensors; call nsa_forward for device tensors")
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    B, H, Tq, D = Q.shape
    Hkv, Tk = K.shape[1], K.shape[2]
    G = H // Hkv
    if out is None:
        out = torch.empty((B, H, Tq, D), dtype=Q.dtype).pin_memory()
    C = _chunk_rows(cfg, Tq, Tk, chunk_rows)
    off = Tk - Tq if cfg.causal else 0
    cur = torch.cuda.current_stream(dev)
    s_in, s_out = _side_streams(dev)
    s_in.wait_stream(cur)
    s_out.wait_stream(cur)

    # Stage 1: every copy in, in the order the units consume them.  The device buffers come from the
    # CURRENT stream's pool of the caching allocator (a side stream's pool would be empty in every call
    # and each buffer a cudaMalloc); the copy stream already waits for everything queued on the current
    # stream so far, and nothing more is queued there until this stage has been issued.
    def dev_empty(shape, dtype):
        t = torch.empty(shape, dtype=dtype, device=dev)
        t.record_stream(s_in)
        return t

    staged = []
    with torch.cuda.device(dev):
        for b in range(B):
            for hk in range(Hkv):
                hs = slice(hk * G, (hk + 1) * G)
                kd = dev_empty((1, 1, Tk, D), K.dtype)
                vd = dev_empty((1, 1, Tk, D), V.dtype)
                k_have = 0
                for c0 in range(0, Tq, C):
                    c1 = min(c0 + C, Tq)
                    k_end = off + c1 if (cfg.causal and C < Tq) else Tk
                    qd = dev_empty((1, G, c1 - c0, D), Q.dtype)
                    gd = dev_empty((1, G, c1 - c0, 3), gate_logits.dtype) if gate_logits is not None else None
                    with torch.cuda.stream(s_in):
                        if k_end > k_have:
                            ops.copy_rows(kd[0, :, k_have:k_end], K[b, hk:hk + 1, k_have:k_end])
                            ops.copy_rows(vd[0, :, k_have:k_end], V[b, hk:hk + 1, k_have:k_end])
                            k_have = k_end
                        ops.copy_rows(qd[0], Q[b, hs, c0:c1])
                        if gd is not None:
                            ops.copy_rows(gd[0], gate_logits[b, hs, c0:c1])
                        ev = torch.cuda.Event()
                        ev.record(s_in)
                    staged.append((b, hs, c0, c1, qd, kd, vd, gd, k_end, ev))

    # stages 2 and 3: compute a unit, send its rows home
    with torch.cuda.device(dev):
        for b, hs, c0, c1, qd, kd, vd, gd, k_end, ev in staged:
            cur.wait_event(ev)
            idx = block_indices_fn(qd, kd[:, :, :k_end]) if block_indices_fn is not None else None
            o = nsa_forward(qd, kd[:, :, :k_end], vd[:, :, :k_end], cfg, gate_logits=gd, block_indices=idx)
            ev2 = torch.cuda.Event()
            ev2.record(cur)
            o.record_stream(s_out)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev2)
                ops.copy_rows(out[b, hs, c0:c1], o[0])
    done = torch.cuda.Event()
    done.record(s_out)          # after the last copy out
    cur.wait_stream(s_out)
    if non_blocking:
        return out, done
    done.synchronize()
    return out


__all__ = ["nsa_forward_host"]
