"""Multi-GPU layouts for the NSA forward: one process per GPU, torch.distributed for the plumbing.

* head parallel (one problem split over the GPUs): (batch, KV head) units are independent -- every kernel's grid
  already factors over them (the reference's grids: nsa/triton/selected.py:288, compressed.py:260, sliding.py:186) --
  so with at most B*Hkv ranks a rank runs the forward on its whole KV heads and nothing is exchanged.  With more
  ranks than units the query heads of a KV head are split over S = ranks / units GPUs; each keeps a replica of the
  KV head.  The only thing the heads of a group share is the block list of a group-shared selection: its score is
  the fp32 sum, in head order, of the heads' block means, so the S ranks all-gather their block means
  ([heads, nq, D], 16-bit: 2 MB at 64k tokens) and every one of them forms the same sum in the same order --
  indices stay bit-exact with the unsplit run, which an all-reduce (another summation order) would not guarantee.
* replicas: every rank runs its own batch element (bench.py --layout replicas); nothing here is needed for it.
* context parallel: query rows are sharded contiguously; rank r owns rows [r*Tl, (r+1)*Tl) of Q,
  the gate logits and the output, and its own slice of K/V.  Causality means it needs the keys of
  ranks <= r, which arrive by ONE all-gather of the raw K/V per tensor over NVLink (NCCL); pooled K/V and the
  block means are then derived locally from the gathered prefix.  The forward is then the ordinary
  one with Tq = Tl and Tk = (r+1)*Tl: queries align with the tail of the keys, which is exactly the
  global causal geometry (offset = r*Tl; nsa/reference.py:57-59,122-126).  The kernels only ever read local HBM.
  Both gathers are started together; the block lists need the keys only and are resolved while the values arrive.
  A collective that does not complete within `timeout_s` raises ContextParallelTimeout instead of blocking.
"""
from __future__ import annotations

import datetime
from dataclasses import dataclass
from typing import Callable, List, Optional, Tuple

import torch
import torch.distributed as dist
from torch import Tensor


def unit_range(n_units: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous, balanced slice [start, end) of `n_units` independent units for `rank`."""
    base, extra = divmod(n_units, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


# ------------------------------------------------------------------ head parallel
@dataclass(frozen=True)
class HeadPartition:
    """What one rank owns of a [B, H, T, D] / [B, Hkv, T, D] problem.  Units are (batch, KV head) pairs numbered
    b*Hkv + hkv.  split == 1: whole units [u0, u1).  split > 1: unit u0 only, query heads [h0, h1) of its group;
    `peers` are the ranks that share the unit, in head order (this rank included)."""
    u0: int
    u1: int
    h0: int
    h1: int
    split: int
    peers: Tuple[int, ...]


def head_partition(B: int, H: int, Hkv: int, world: int, rank: int) -> HeadPartition:
    units, G = B * Hkv, H // Hkv
    if world <= units:
        u0, u1 = unit_range(units, world, rank)
        return HeadPartition(u0, u1, 0, G, 1, (rank,))
    if world % units or G % (world // units):
        raise ValueError(f"{world} ranks cannot split {units} (batch, KV head) units of {G} query heads evenly")
    S = world // units
    u, part = divmod(rank, S)
    return HeadPartition(u, u + 1, part * (G // S), (part + 1) * (G // S), S, tuple(u * S + j for j in range(S)))


def head_groups(B: int, H: int, Hkv: int, world: int, rank: int):
    """The process group of the ranks that share this rank's KV head (None when nothing is shared).  Collective:
    every rank of the default group must call it, with the same arguments."""
    part = head_partition(B, H, Hkv, world, rank)
    if part.split == 1:
        return None
    mine = None
    for u in range(B * Hkv):
        g = dist.new_group([u * part.split + j for j in range(part.split)])
        if u == part.u0:
            mine = g
    return mine


def shard_heads(Q: Tensor, K: Tensor, V: Tensor, part: HeadPartition, gate_logits: Optional[Tensor] = None):
    """This rank's slices as a batch-1 problem: Q/gates [1, heads, Tq, .], K/V [1, kv heads, Tk, D] (views when the
    inputs are dense)."""
    B, H, Tq, D = Q.shape
    Hkv, Tk = K.shape[1], K.shape[2]
    G = H // Hkv
    n = part.u1 - part.u0
    Qu = Q.reshape(B * Hkv, G, Tq, D)[part.u0:part.u1, part.h0:part.h1].reshape(1, n * (part.h1 - part.h0), Tq, D)
    Ku = K.reshape(B * Hkv, 1, Tk, D)[part.u0:part.u1].reshape(1, n, Tk, D)
    Vu = V.reshape(B * Hkv, 1, Tk, D)[part.u0:part.u1].reshape(1, n, Tk, D)
    gu = None
    if gate_logits is not None:
        gu = gate_logits.reshape(B * Hkv, G, Tq, 3)[part.u0:part.u1, part.h0:part.h1].reshape(1, n * (part.h1 - part.h0), Tq, 3)
    return Qu, Ku, Vu, gu


def shard_kv_heads(Q: Tensor, K: Tensor, V: Tensor, world: int, rank: int, gate_logits: Optional[Tensor] = None):
    """Whole-unit slices for `rank` of `world` (at most B*Hkv ranks)."""
    B, H = Q.shape[0], Q.shape[1]
    return shard_heads(Q, K, V, head_partition(B, H, K.shape[1], min(world, B * K.shape[1]), rank), gate_logits)


def gather_heads(x_local: Tensor, group) -> Tensor:
    """[1, h, ...] per rank -> [1, S*h, ...] in rank (= head) order, identical on every rank of `group`."""
    S = dist.get_world_size(group)
    x_local = x_local.contiguous()
    flat = torch.empty((S * x_local.shape[0],) + tuple(x_local.shape[1:]), dtype=x_local.dtype, device=x_local.device)
    dist.all_gather_into_tensor(flat, x_local, group=group)           # rank-major along dim 0
    buf = flat.view((S,) + tuple(x_local.shape))
    return buf.transpose(0, 1).reshape((x_local.shape[0], S * x_local.shape[1]) + tuple(x_local.shape[2:]))


def resolve_block_indices_split(Q_local: Tensor, K_local: Tensor, cfg, group, *, scale: float) -> Tensor:
    """Block lists for a rank that holds only some query heads of its KV head.  One list per query head: local.
    One list per KV head (cfg.select_per_group): the heads' block means are all-gathered over `group` and summed
    by the selection kernel in head order, exactly as on one GPU."""
    from . import ops
    from .forward import _cfg
    bm, bn = int(cfg.block_size_m), int(cfg.block_size_n)
    Qb = ops.pool_mean(Q_local.detach(), bm)
    Kb = ops.pool_mean(K_local.detach(), bn)
    shared = bool(_cfg(cfg, "select_per_group", False))
    if shared and group is not None:
        Qb = gather_heads(Qb, group)
    nq, nk = Qb.shape[2], Kb.shape[2]
    return ops.select_blocks_from_means(Qb, Kb, top_k=int(cfg.top_k), bm=bm, bn=bn, offset=nk * bn - nq * bm,
                                        causal=bool(cfg.causal), scale=float(scale), force_first=_cfg(cfg, "force_first", 0),
                                        force_local=_cfg(cfg, "force_local", 0), shared_per_group=shared)


def nsa_forward_head_parallel(Q_local: Tensor, K_local: Tensor, V_local: Tensor, cfg, *, gate_logits: Optional[Tensor] = None,
                              group=None) -> Tensor:
    """NSA forward on this rank's heads (shard_heads).  `group`: the ranks sharing this rank's KV head
    (head_groups), None when the rank owns whole KV heads.  Inference route (no autograd)."""
    from .forward import nsa_forward
    if group is None:
        return nsa_forward(Q_local, K_local, V_local, cfg, gate_logits=gate_logits)
    D = Q_local.shape[-1]
    scale = cfg.scale if cfg.scale is not None else 1.0 / (D ** 0.5)
    idx = resolve_block_indices_split(Q_local, K_local, cfg, group, scale=float(scale))
    return nsa_forward(Q_local, K_local, V_local, cfg, gate_logits=gate_logits, block_indices=idx)


# ------------------------------------------------------------------ context parallel
class ContextParallelTimeout(RuntimeError):
    """A collective of the context-parallel layout did not complete in time (a rank is late or gone)."""


class _PrefixGather:
    """One all-gather of [B,Hkv,Tl,D] shards along the sequence, started at construction, finished by `wait()`."""

    def __init__(self, x_local: Tensor, group=None, stats: Optional[dict] = None):
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.x = x_local.contiguous()
        self.work = None
        if self.world > 1:
            B, Hkv, Tl, D = self.x.shape
            self.flat = torch.empty((self.world * B, Hkv, Tl, D), dtype=self.x.dtype, device=self.x.device)
            self.work = dist.all_gather_into_tensor(self.flat, self.x, group=group, async_op=True)
            if stats is not None:
                stats["bytes_received"] = stats.get("bytes_received", 0) + (self.world - 1) * self.x.numel() * self.x.element_size()

    def wait(self, timeout_s: Optional[float] = None) -> Tensor:
        """The causal prefix this rank needs, [B,Hkv,(rank+1)*Tl,D] contiguous: the collective's buffer laid out
        head-major by a single strided copy of the (rank+1)/world part that is needed.  With `timeout_s` the
        collective is waited for on the host and ContextParallelTimeout is raised if it has not completed by then;
        without, the current stream waits for it and the host goes on."""
        if self.work is None:
            return self.x
        try:
            ok = self.work.wait(datetime.timedelta(seconds=timeout_s)) if timeout_s is not None else self.work.wait()
        except RuntimeError as e:
            raise ContextParallelTimeout(f"all-gather of the key prefix did not complete within {timeout_s} s: {e}") from e
        if ok is False:
            raise ContextParallelTimeout(f"all-gather of the key prefix did not complete within {timeout_s} s")
        B, Hkv, Tl, D = self.x.shape
        buf = self.flat.view(self.world, B, Hkv, Tl, D)
        return buf[: self.rank + 1].permute(1, 2, 0, 3, 4).reshape(B, Hkv, (self.rank + 1) * Tl, D)


def gather_key_prefix(x_local: Tensor, group=None, *, timeout_s: Optional[float] = None, stats: Optional[dict] = None) -> Tensor:
    """All-gather [B,Hkv,Tl,D] shards along the sequence and return the causal prefix this rank
    needs, [B,Hkv,(rank+1)*Tl,D] contiguous.  One collective into one preallocated buffer.  `timeout_s`: see
    _PrefixGather.wait."""
    return _PrefixGather(x_local, group, stats).wait(timeout_s)


def nsa_forward_context_parallel(Q_local: Tensor, K_local: Tensor, V_local: Tensor, cfg, *,
                                 gate_logits: Optional[Tensor] = None, group=None,
                                 forward_fn: Optional[Callable] = None, timeout_s: Optional[float] = None,
                                 stats: Optional[dict] = None) -> Tensor:
    """Causal NSA forward with the sequence sharded contiguously over the ranks of `group`.
    Inputs are this rank's shards ([B,H,Tl,D], [B,Hkv,Tl,D]); returns this rank's output shard.
    Both all-gathers are started at once.  With the default forward and block-mean selection, the block lists -- which
    need the keys only -- are resolved while the values are still arriving (the collectives run on the library's own
    stream; the pooling and selection kernels on the caller's).  `forward_fn(Q, K, V, cfg, gate_logits=...)` replaces
    the forward (then nothing is overlapped).  `stats` (a dict) receives the bytes this rank received; `timeout_s`:
    see _PrefixGather.wait."""
    if not cfg.causal:
        raise ValueError("context-parallel layout is defined for causal attention")
    gk = _PrefixGather(K_local, group, stats)
    gv = _PrefixGather(V_local, group, stats)
    K_pref = gk.wait(timeout_s)
    if forward_fn is not None:
        return forward_fn(Q_local, K_pref, gv.wait(timeout_s), cfg, gate_logits=gate_logits)
    from .forward import _cfg, _resolve_block_indices, nsa_forward
    idx = None
    if _cfg(cfg, "scorer", "mean") == "mean" and Q_local.is_cuda:
        D = Q_local.shape[-1]
        scale = cfg.scale if cfg.scale is not None else 1.0 / (D ** 0.5)
        idx = _resolve_block_indices(Q_local, K_pref, block_size_m=cfg.block_size_m, block_size_n=cfg.block_size_n,
                                     top_k=cfg.top_k, causal=cfg.causal, scale=float(scale),
                                     force_first=_cfg(cfg, "force_first", 0), force_local=_cfg(cfg, "force_local", 0),
                                     shared_per_group=bool(_cfg(cfg, "select_per_group", False)))
    return nsa_forward(Q_local, K_pref, gv.wait(timeout_s), cfg, gate_logits=gate_logits, block_indices=idx)


__all__ = ["unit_range", "HeadPartition", "head_partition", "head_groups", "shard_heads", "shard_kv_heads", "gather_heads",
           "resolve_block_indices_split", "nsa_forward_head_parallel", "ContextParallelTimeout", "gather_key_prefix",
           "nsa_forward_context_parallel"]
