"""Drop-in shim: after `install()`, the module names the reference's callers import
(`nsa.triton.compressed|selected|sliding|gating|forward|backward|fp8|moba`, `nsa.cuda`) resolve to
this package, so the reference's model, benchmarks and tests run on these kernels unchanged.
`nsa.reference` (and everything else under `nsa`) still comes from the reference checkout
when it is importable; otherwise a minimal `nsa.reference` with NSAConfig is provided."""
from __future__ import annotations

import importlib
import sys
import types

_MAP = {
    "nsa.triton.compressed": "compressed", "nsa.triton.selected": "selected", "nsa.triton.sliding": "sliding",
    "nsa.triton.gating": "gating", "nsa.triton.forward": "forward", "nsa.triton.backward": "backward",
    "nsa.triton.fp8": "fp8", "nsa.triton.moba": "moba", "nsa.cuda": "native",
}


def install(fuse_caller: bool = False) -> None:
    """`fuse_caller`: also give the reference's attention module (nsa/model/llama_nsa.py:67-96), when it is
    importable, the token-major forward -- rotary embedding and head-major re-layout in one pass per tensor,
    gate logits and output in the module's own [B,T,...] layouts -- for CUDA inputs outside autograd; every
    other call still runs the module's own code."""
    pkg = __name__.rsplit(".", 1)[0]
    try:
        importlib.import_module("nsa")
    except ImportError:
        nsa = types.ModuleType("nsa")
        nsa.__path__ = []
        sys.modules["nsa"] = nsa
        ref = types.ModuleType("nsa.reference")
        ref.NSAConfig = importlib.import_module(pkg + ".config").NSAConfig
        sys.modules["nsa.reference"] = ref
    if "nsa.triton" not in sys.modules:
        tri = types.ModuleType("nsa.triton")
        tri.__path__ = []
        sys.modules["nsa.triton"] = tri
    for name, ours in _MAP.items():
        mod = importlib.import_module(f"{pkg}.{ours}")
        sys.modules[name] = mod
        parent, _, leaf = name.rpartition(".")
        setattr(sys.modules[parent], leaf, mod)
    if fuse_caller:
        _patch_attention_module(pkg)


def _patch_attention_module(pkg: str) -> None:
    try:
        llama = importlib.import_module("nsa.model.llama_nsa")
    except ImportError:
        return
    cls = llama.NSAAttention
    if getattr(cls.forward, "_b200_token_major", False):
        return
    import torch
    layer = importlib.import_module(pkg + ".layer")
    original = cls.forward

    def forward(self, x, cos, sin):
        needs_grad = torch.is_grad_enabled() and (x.requires_grad or any(p.requires_grad for p in self.parameters()))
        if not x.is_cuda or needs_grad or self.nsa_cfg.pool != "mean":
            return original(self, x, cos, sin)
        B, T, _ = x.shape
        H, D = self.cfg.n_heads, self.cfg.head_dim
        q = self.q_proj(x).view(B, T, H, D)
        k = self.k_proj(x).view(B, T, H, D)
        v = self.v_proj(x).view(B, T, H, D)
        gates = self.gate(x).view(B, T, H, 3)
        out = layer.nsa_attention_token_major(q, k, v, cos, sin, self.nsa_cfg, gate_logits=gates)
        return self.o_proj(out.to(x.dtype))

    forward._b200_token_major = True
    cls.forward = forward
