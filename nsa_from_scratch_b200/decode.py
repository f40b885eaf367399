"""Decoding against a KV cache: the Tq << Tk case of the forward.

Every function of the path already takes Tq < Tk with the queries aligned to the tail of the keys
(`offset = Tk - Tq`, nsa/reference.py:57-59); what a decoder adds is a cache that grows in place.  The cache
keeps, next to K and V, the two derived tensors the forward recomputes from scratch on every call -- the
pooled K/V of the compressed branch and the block means the selection scores against -- and brings them up
to date from the appended rows only.  The kernels are handed the whole allocation as "the" K/V tensor
together with the true offsets: under the causal rules no row past the filled length is ever visible, so no
copy of the filled prefix is made.  (Rows past the filled length are still multiplied by zero weights: the
cache starts zero-filled so that they are finite.)
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import Tensor

from . import _lib as L
from . import ops
from .forward import _cfg


def _cdiv(a: int, b: int) -> int:
    return (a + b - 1) // b


class KVCache:
    """K, V [B,Hkv,max_len,D] with `length` rows filled, pooled K/V and selection block means kept current."""

    def __init__(self, B: int, Hkv: int, D: int, max_len: int, cfg, dtype: torch.dtype = torch.bfloat16, device="cuda"):
        if not cfg.causal:
            raise ValueError("KVCache: decoding needs causal=True")
        self.cfg = cfg
        self.bc = int(cfg.block_size_c)
        self.stride = self.bc if getattr(cfg, "stride_c", None) is None else int(cfg.stride_c)
        self.bn = int(cfg.block_size_n)
        self.max_len = int(max_len)
        z = lambda n: torch.zeros((B, Hkv, n, D), dtype=dtype, device=device)
        self.K, self.V = z(max_len), z(max_len)
        self.Kc, self.Vc = z(max(1, self.n_pooled(max_len))), z(max(1, self.n_pooled(max_len)))
        self.Kb = z(_cdiv(max_len, self.bn))
        self.length = 0
        self.filled_dev: Optional[Tensor] = None    # device copy of `length`, kept once a GraphedDecoder asks for it

    def n_pooled(self, T: int) -> int:
        if self.stride == self.bc:
            return _cdiv(T, self.bc)
        return 0 if T < self.bc else (T - self.bc) // self.stride + 1

    def reset(self) -> None:
        self._set_length(0)

    def _set_length(self, n: int) -> None:
        self.length = n
        if self.filled_dev is not None:
            self.filled_dev.fill_(n)

    def append(self, k: Tensor, v: Tensor) -> None:
        """k, v [B,Hkv,t,D]: the next t positions."""
        t = k.shape[2]
        T0, T1 = self.length, self.length + t
        if T1 > self.max_len:
            raise ValueError(f"KVCache: {T1} rows exceed the allocation of {self.max_len}")
        k, v = k.contiguous(), v.contiguous()
        B, Hkv, _, D = self.K.shape
        if k.shape != (B, Hkv, t, D) or v.shape != k.shape or k.dtype != self.K.dtype or v.dtype != self.K.dtype:
            raise ValueError(f"KVCache.append: expected [{B},{Hkv},t,{D}] {self.K.dtype} tensors, got {tuple(k.shape)} {k.dtype}")
        # one launch: rows into K/V, and every pooled window / selection-block mean that contains a new row
        with torch.cuda.device(self.K.device):
            L.check(L.load().nsa_cache_append(k.data_ptr(), v.data_ptr(), self.K.data_ptr(), self.V.data_ptr(), self.Kc.data_ptr(),
                                              self.Vc.data_ptr(), self.Kb.data_ptr(), B, Hkv, D, t, T0, self.max_len,
                                              self.Kc.shape[2], self.Kb.shape[2], self.bc, self.stride, self.bn,
                                              L.dtype_code(self.K.dtype), L.stream_ptr()), "nsa_cache_append")
        self._set_length(T1)


def _split_ways(B: int, H: int, Hkv: int, Tq: int, n_pooled: int) -> int:
    """Thread blocks per work item of the attention launch: enough to reach every SM once when there are few
    work items, but at least two 128-key tiles of the compressed branch (the long one) per block."""
    G = H // Hkv
    gh = 4 if G % 4 == 0 else (2 if G % 2 == 0 else 1)
    items = B * Hkv * (G // gh) * _cdiv(_cdiv(Tq, 64), 4 // gh)
    sms = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    return max(1, min(sms // max(items, 1), _cdiv(n_pooled, 128) // 2, 16))


def nsa_decode(q: Tensor, cache: KVCache, *, gate_logits: Optional[Tensor] = None, nsplit: Optional[int] = None) -> Tensor:
    """q [B,H,Tq,D]: the queries of the LAST Tq cached positions (append their keys first).  Returns
    [B,H,Tq,D] -- what `nsa_forward(q, K[:, :, :length], V[:, :, :length], cfg)` returns.  `nsplit`: thread
    blocks per work item of the attention launch (None: chosen from the sizes; 1: the ordinary launch)."""
    cfg = cache.cfg
    B, H, Tq, D = q.shape
    Tk = cache.length
    if Tq > Tk:
        raise ValueError(f"nsa_decode: {Tq} queries but only {Tk} cached positions")
    scale = float(cfg.scale if cfg.scale is not None else 1.0 / (D ** 0.5))
    bm, bn = int(cfg.block_size_m), cache.bn
    Qb = ops.pool_mean(q, bm, bm)
    idx = ops.select_blocks_from_means(
        Qb, cache.Kb, top_k=cfg.top_k, bm=bm, bn=bn, offset=_cdiv(Tk, bn) * bn - _cdiv(Tq, bm) * bm, causal=True, scale=scale,
        force_first=_cfg(cfg, "force_first", 0), force_local=_cfg(cfg, "force_local", 0),
        shared_per_group=bool(_cfg(cfg, "select_per_group", False)))
    Tk_pad = _cdiv(Tk, cache.bc) * cache.bc if cache.stride == cache.bc else Tk
    out, _ = ops.attention_fwd(
        q, cache.K, cache.V, branches=L.BRANCH_COMPRESSED | L.BRANCH_SELECTED | L.BRANCH_SLIDING, fused=True, causal=True,
        scale=scale, Kc=cache.Kc, Vc=cache.Vc, cmp_block=cache.bc, cmp_stride=cache.stride, cmp_offset=Tk_pad - Tq,
        idx=idx, bm=bm, bn=bn, window=cfg.window_size, gates=gate_logits,
        gate_act=L.GATE_SOFTMAX if cfg.gate_activation == "softmax" else L.GATE_SIGMOID, offset=Tk - Tq,
        nsplit=_split_ways(B, H, cache.K.shape[1], Tq, cache.n_pooled(Tk)) if nsplit is None else int(nsplit))
    return out


class GraphedDecoder:
    """A decoding step -- append the new keys/values, block means of the new queries, selection, split attention
    launch and merge -- captured once into a CUDA graph and replayed for every step.  The cache's fill count
    lives in device memory and every length-dependent quantity is derived there, so the same graph serves the
    whole generation.  Fill `q`, `k`, `v` (and `gate_logits`) in place, call `step()`, read `out`."""

    def __init__(self, cache: KVCache, n_heads: int, *, tokens_per_step: int = 1, gates: bool = True,
                 nsplit: Optional[int] = None):
        cfg = cache.cfg
        B, Hkv, _, D = cache.K.shape
        dev, dt = cache.K.device, cache.K.dtype
        self.cache, self.t = cache, int(tokens_per_step)
        self.q = torch.zeros((B, n_heads, self.t, D), dtype=dt, device=dev)
        self.k = torch.zeros((B, Hkv, self.t, D), dtype=dt, device=dev)
        self.v = torch.zeros((B, Hkv, self.t, D), dtype=dt, device=dev)
        self.gate_logits = torch.zeros((B, n_heads, self.t, 3), dtype=torch.float32, device=dev) if gates else None
        if cache.filled_dev is None:
            cache.filled_dev = torch.full((1,), cache.length, dtype=torch.int32, device=dev)
        # the grid is part of the graph: split as for a full cache
        self.nsplit = _split_ways(B, n_heads, Hkv, self.t, cache.n_pooled(cache.max_len)) if nsplit is None else int(nsplit)
        self.scale = float(cfg.scale if cfg.scale is not None else 1.0 / (D ** 0.5))
        start = cache.length
        if start + self.t > cache.max_len:
            raise ValueError("GraphedDecoder: the cache has no room for a step")
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for _ in range(2):                     # warm-up steps write past the filled rows; the count is put back
                self._launches()
                cache.filled_dev.fill_(start)
        torch.cuda.current_stream(dev).wait_stream(side)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.out = self._launches()
        cache.filled_dev.fill_(start)              # capturing runs nothing; be explicit all the same

    def _launches(self) -> Tensor:
        c, cfg = self.cache, self.cache.cfg
        B, Hkv, _, D = c.K.shape
        H = self.q.shape[1]
        bm = int(cfg.block_size_m)
        lib = L.load()
        with torch.cuda.device(c.K.device):
            L.check(lib.nsa_cache_append_dev(self.k.data_ptr(), self.v.data_ptr(), c.K.data_ptr(), c.V.data_ptr(), c.Kc.data_ptr(),
                                             c.Vc.data_ptr(), c.Kb.data_ptr(), B, Hkv, D, self.t, c.filled_dev.data_ptr(), c.max_len,
                                             c.Kc.shape[2], c.Kb.shape[2], c.bc, c.stride, c.bn, L.dtype_code(c.K.dtype),
                                             L.stream_ptr()), "nsa_cache_append_dev")
            Qb = ops.pool_mean(self.q, bm, bm)
            shared = bool(_cfg(cfg, "select_per_group", False))
            nq = Qb.shape[2]
            idx = torch.empty((B, Hkv if shared else H, nq, min(cfg.top_k, c.Kb.shape[2])), device=c.K.device, dtype=torch.int32)
            L.check(lib.nsa_select_blocks_cached(Qb.data_ptr(), c.Kb.data_ptr(), idx.data_ptr(), B, H, Hkv, nq, c.Kb.shape[2], D,
                                                 cfg.top_k, bm, c.bn, c.filled_dev.data_ptr(), self.scale,
                                                 _cfg(cfg, "force_first", 0), _cfg(cfg, "force_local", 0), int(shared),
                                                 L.dtype_code(Qb.dtype), L.stream_ptr()), "nsa_select_blocks_cached")
        out, _ = ops.attention_fwd(
            self.q, c.K, c.V, branches=L.BRANCH_COMPRESSED | L.BRANCH_SELECTED | L.BRANCH_SLIDING, fused=True, causal=True,
            scale=self.scale, Kc=c.Kc, Vc=c.Vc, cmp_block=c.bc, cmp_stride=c.stride, cmp_offset=0, idx=idx, bm=bm, bn=c.bn,
            window=cfg.window_size, gates=self.gate_logits,
            gate_act=L.GATE_SOFTMAX if cfg.gate_activation == "softmax" else L.GATE_SIGMOID, offset=0,
            nsplit=self.nsplit, dyn_len=c.filled_dev)
        return out

    def step(self) -> Tensor:
        c = self.cache
        if c.length + self.t > c.max_len:
            raise ValueError(f"GraphedDecoder: {c.length} + {self.t} rows exceed the allocation of {c.max_len}")
        self.graph.replay()
        c.length += self.t                         # the device count was advanced by the graph
        return self.out


__all__ = ["KVCache", "nsa_decode", "GraphedDecoder"]
