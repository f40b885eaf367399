"""Multi-GPU layouts for the NSA forward: one process per GPU, torch.distributed for the plumbing.

* batch x KV-head parallel: (batch, KV head) units are independent, every kernel's grid already
  factors over them, so a rank simply runs the forward on its slice -- no collective.
* context parallel: query rows are sharded contiguously; rank r owns rows [r*Tl, (r+1)*Tl) of Q,
  the gate logits and the output, and its own slice of K/V.  Causality means it needs the keys of
  ranks <= r, which arrive by ONE all-gather of the raw K/V over NVLink (NCCL); pooled K/V and the
  block means are then derived locally from the gathered prefix.  The forward is then the ordinary
  one with Tq = Tl and Tk = (r+1)*Tl: queries align with the tail of the keys, which is exactly the
  global causal geometry (offset = r*Tl).  The kernels only ever read local HBM.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist
from torch import Tensor


def unit_range(n_units: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous, balanced slice [start, end) of `n_units` independent units for `rank`."""
    base, extra = divmod(n_units, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def shard_kv_heads(Q: Tensor, K: Tensor, V: Tensor, world: int, rank: int, gate_logits: Optional[Tensor] = None):
    """Slices of Q/K/V (and gate logits) holding this rank's (batch, KV head) units.  Units are
    numbered b*Hkv + hkv; a rank gets whole KV heads together with their query-head groups, so block
    lists shared per group stay local.  Returns (Q, K, V, gates) with the batch and head axes merged
    into the head axis of a batch-1 problem."""
    B, H, Tq, D = Q.shape
    Hkv = K.shape[1]
    G = H // Hkv
    u0, u1 = unit_range(B * Hkv, world, rank)
    Qu = Q.reshape(B * Hkv, G, Tq, D)[u0:u1].reshape(1, (u1 - u0) * G, Tq, D)
    Ku = K.reshape(B * Hkv, 1, K.shape[2], D)[u0:u1].reshape(1, u1 - u0, K.shape[2], D)
    Vu = V.reshape(B * Hkv, 1, V.shape[2], D)[u0:u1].reshape(1, u1 - u0, V.shape[2], D)
    gu = None
    if gate_logits is not None:
        gu = gate_logits.reshape(B * Hkv, G, Tq, 3)[u0:u1].reshape(1, (u1 - u0) * G, Tq, 3)
    return Qu, Ku, Vu, gu


def gather_key_prefix(x_local: Tensor, group=None) -> Tensor:
    """All-gather [B,Hkv,Tl,D] shards along the sequence and return the causal prefix this rank
    needs, [B,Hkv,(rank+1)*Tl,D] contiguous."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    if world == 1:
        return x_local.contiguous()
    parts = [torch.empty_like(x_local) for _ in range(world)]
    dist.all_gather(parts, x_local.contiguous(), group=group)
    return torch.cat(parts[: rank + 1], dim=2)


def nsa_forward_context_parallel(Q_local: Tensor, K_local: Tensor, V_local: Tensor, cfg, *,
                                 gate_logits: Optional[Tensor] = None, group=None,
                                 forward_fn: Optional[Callable] = None) -> Tensor:
    """Causal NSA forward with the sequence sharded contiguously over the ranks of `group`.
    Inputs are this rank's shards ([B,H,Tl,D], [B,Hkv,Tl,D]); returns this rank's output shard.
    `forward_fn(Q, K, V, cfg, gate_logits=...)` defaults to `nsa_forward`."""
    if not cfg.causal:
        raise ValueError("context-parallel layout is defined for causal attention")
    if forward_fn is None:
        from .forward import nsa_forward as forward_fn
    K_pref = gather_key_prefix(K_local, group)
    V_pref = gather_key_prefix(V_local, group)
    return forward_fn(Q_local, K_pref, V_pref, cfg, gate_logits=gate_logits)


__all__ = ["unit_range", "shard_kv_heads", "gather_key_prefix", "nsa_forward_context_parallel"]
