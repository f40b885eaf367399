"""Generate the golden fixtures in this directory from the reference project.

Run once, in a container where the reference checkout is importable:

    python tests/golden/make_golden.py --reference /path/to/nsa-from-scratch

Every case stores its seeded inputs and the outputs of the REFERENCE's own
functions (nsa/reference.py, nsa/triton/forward.py, nsa/triton/fp8.py,
nsa/triton/gating.py -- all plain torch, they run on CPU).  The fixtures are
what pins the CPU oracle (tests/test_oracle_golden.py) and, through it, the
CUDA kernels.  Tensors are saved as fp32 / int32 numpy arrays; bf16 inputs
are saved after rounding, so `.to(bfloat16)` restores them exactly.
"""

from __future__ import annotations

import argparse
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def qkv(seed, B, H, Tq, Tk, D, dtype, amp=1.0):
    g = torch.Generator().manual_seed(seed)
    Q = (torch.randn(B, H, Tq, D, generator=g) * amp).to(dtype)
    K = (torch.randn(B, H, Tk, D, generator=g) * amp).to(dtype)
    V = (torch.randn(B, H, Tk, D, generator=g) * amp).to(dtype)
    return Q, K, V, g


def np32(t):
    return t.detach().float().numpy()


def layer_cases():
    """The reference's attention module (nsa/model/llama_nsa.py) on CPU: its fp32 route through
    nsa_attention_reference, plus the rotary embedding on its own.  top_k covers every legal block so the
    fp32 scorer and a 16-bit scorer cannot disagree on the selection."""
    from nsa.model.config import TransformerConfig
    from nsa.model.llama_dense import _apply_rope, _build_rope_cache
    from nsa.model.llama_nsa import NSAAttention
    out, meta = {}, []
    for name, (B, T, H, D, hidden, bc, k, W, act) in {
        "layer_a": (1, 320, 4, 64, 128, 32, 8, 96, "sigmoid"),
        "layer_b": (1, 256, 2, 128, 64, 64, 4, 64, "softmax"),
    }.items():
        torch.manual_seed(71)
        cfg = TransformerConfig(n_heads=H, head_dim=D, hidden_size=hidden, nsa_block_size_c=bc, nsa_top_k=k,
                                nsa_window_size=W, nsa_gate_activation=act)
        mod = NSAAttention(cfg).float()
        g = torch.Generator().manual_seed(72)
        x = torch.randn(B, T, hidden, generator=g)
        cos, sin = _build_rope_cache(T, D, cfg.rope_theta, "cpu", torch.float32)
        with torch.no_grad():
            y = mod(x, cos, sin)
            q = mod.q_proj(x).view(B, T, H, D)
            kk = mod.k_proj(x).view(B, T, H, D)
            qr, kr = _apply_rope(q.transpose(1, 2), kk.transpose(1, 2), cos, sin)
        out.update({f"{name}.x": np32(x), f"{name}.cos": np32(cos), f"{name}.sin": np32(sin), f"{name}.y": np32(y)})
        if name == "layer_a":      # the rotary embedding on its own: projection output in, _apply_rope out
            out.update({f"{name}.q_bthd": np32(q), f"{name}.q_rope": np32(qr)})
        for pn, pv in mod.state_dict().items():
            out[f"{name}.w.{pn}"] = np32(pv)
        meta.append((name, dict(B=B, T=T, H=H, D=D, hidden=hidden, bc=bc, top_k=k, W=W, act=act)))
    np.savez_compressed(os.path.join(HERE, "layer_golden.npz"), **out)
    with open(os.path.join(HERE, "layer_golden.meta.txt"), "w") as f:
        f.write(f"torch {torch.__version__}\n")
        for n, m in meta:
            f.write(f"{n}: {m}\n")
    print("wrote", len(out), "arrays (layer)")


def learned_pool_cases():
    """Learned pooling: the reference's plain-torch compressed branch and combined forward with pool="learned"
    (nsa/reference.py:109-113, 288-347), its only implementation of that option."""
    from nsa import reference as R
    out, meta = {}, []
    for name, (B, H, Tq, Tk, D, bc, causal) in {"lp_a": (1, 2, 128, 128, 64, 32, True), "lp_b": (1, 2, 96, 200, 64, 64, True)}.items():
        Q, K, V, g = qkv(81, B, H, Tq, Tk, D, torch.bfloat16)
        pk = torch.randn(bc, D, generator=g) / D ** 0.5
        pv = torch.randn(bc, D, generator=g) / D ** 0.5
        o, l = R.compressed_attention_reference(Q.float(), K.float(), V.float(), block_size_c=bc, pool="learned",
                                                pool_proj_k=pk, pool_proj_v=pv, causal=causal)
        out.update({f"{name}.Q": np32(Q), f"{name}.K": np32(K), f"{name}.V": np32(V), f"{name}.pk": np32(pk), f"{name}.pv": np32(pv),
                    f"{name}.out": np32(o), f"{name}.lse": np32(l)})
        meta.append((name, dict(B=B, H=H, Tq=Tq, Tk=Tk, D=D, bc=bc, causal=causal)))
    # combined forward with learned pooling (geometry 32/32/32, top-3, window 48, as the other combined cases)
    Q, K, V, g = qkv(82, 1, 2, 128, 128, 64, torch.bfloat16)
    gates = torch.randn(1, 2, 128, 3, generator=g)
    pk = torch.randn(32, 64, generator=g) / 8.0
    pv = torch.randn(32, 64, generator=g) / 8.0
    cfg = R.NSAConfig(block_size_c=32, block_size_n=32, block_size_m=32, top_k=3, window_size=48, pool="learned")
    o = R.nsa_attention_reference(Q.float(), K.float(), V.float(), cfg, gates=gates, pool_proj_k=pk, pool_proj_v=pv)
    out.update({"lp_nsa.Q": np32(Q), "lp_nsa.K": np32(K), "lp_nsa.V": np32(V), "lp_nsa.gates": np32(gates), "lp_nsa.pk": np32(pk),
                "lp_nsa.pv": np32(pv), "lp_nsa.out": np32(o)})
    np.savez_compressed(os.path.join(HERE, "learned_pool_golden.npz"), **out)
    print("wrote", len(out), "arrays (learned pooling)")


def moba_cases():
    """MoBA routing: the reference's per-query top-k block lists (nsa/triton/moba.py:18-92, plain torch)."""
    from nsa.triton.moba import _per_query_top_k_indices
    out = {}
    for name, (B, H, Tq, Tk, D, kq, cap, causal) in {"moba_a": (1, 2, 1024, 1024, 64, 4, 8, True),
                                                     "moba_b": (1, 2, 1024, 1024, 64, 8, 6, True),      # unions overflow the cap
                                                     "moba_c": (1, 2, 512, 768, 64, 3, 16, False)}.items():
        Q, K, V, g = qkv(91, B, H, Tq, Tk, D, torch.bfloat16)
        idx = _per_query_top_k_indices(Q, K, block_size_n=64, block_size_m=64, top_k_per_query=kq, top_k_cap=cap,
                                       causal=causal, scale=D ** -0.5)
        out.update({f"{name}.Q": np32(Q), f"{name}.K": np32(K), f"{name}.idx": idx.numpy().astype(np.int32),
                    f"{name}.par": np.array([kq, cap, int(causal)], dtype=np.int32)})
    np.savez_compressed(os.path.join(HERE, "moba_golden.npz"), **out)
    print("wrote", len(out), "arrays (moba routing)")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of the reference checkout")
    ap.add_argument("--part", default="all", choices=["all", "kernels", "layer", "learned", "moba"],
                    help="kernels: reference_golden.npz; layer: layer_golden.npz; learned: learned_pool_golden.npz; moba: moba_golden.npz")
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    sys.path.insert(0, os.path.join(HERE, "..", ".."))
    if args.part in ("all", "layer"):
        layer_cases()
    if args.part in ("all", "learned"):
        learned_pool_cases()
    if args.part in ("all", "moba"):
        moba_cases()
    if args.part in ("layer", "learned", "moba"):
        return
    from nsa import reference as R
    from nsa.triton import forward as F_
    from nsa.triton import fp8 as FP8
    from nsa.triton import gating as GT
    from nsa.triton.selected import _topk_indices_from_scores
    from oracle import nsa_oracle as O

    out = {}
    meta = []

    # ---- compressed ------------------------------------------------------
    for name, (B, H, Tq, Tk, D, bc, causal, dt) in {
        "cmp_a": (1, 2, 128, 128, 32, 32, True, torch.float32),
        "cmp_b": (1, 2, 96, 200, 32, 64, True, torch.bfloat16),     # ragged, Tq < Tk
        "cmp_c": (2, 2, 128, 192, 64, 32, False, torch.bfloat16),
    }.items():
        Q, K, V, _ = qkv(11, B, H, Tq, Tk, D, dt, 0.5)
        o, l = R.compressed_attention_reference(Q.float(), K.float(), V.float(),
                                                block_size_c=bc, causal=causal)
        # pooled keys in the INPUT dtype, as the kernels' wrapper pools them
        from nsa.triton.compressed import _mean_pool
        out.update({f"{name}.Q": np32(Q), f"{name}.K": np32(K), f"{name}.V": np32(V),
                    f"{name}.out": np32(o), f"{name}.lse": np32(l),
                    f"{name}.Kc": np32(_mean_pool(K, bc))})
        meta.append((name, dict(B=B, H=H, Tq=Tq, Tk=Tk, D=D, bc=bc, causal=causal,
                                dtype=str(dt))))

    # ---- scorer / top-k ---------------------------------------------------
    for name, (B, H, Tq, Tk, D, bm, bn, k, causal, dt) in {
        "sel_idx_a": (1, 2, 512, 512, 32, 64, 64, 4, True, torch.bfloat16),
        "sel_idx_b": (1, 2, 200, 456, 32, 32, 32, 5, True, torch.bfloat16),   # ragged
        "sel_idx_c": (1, 2, 256, 256, 64, 64, 64, 3, False, torch.float16),
    }.items():
        Q, K, V, _ = qkv(23, B, H, Tq, Tk, D, dt)
        s = 1.0 / D ** 0.5
        idx = F_._resolve_block_indices(Q, K, block_size_m=bm, block_size_n=bn, top_k=k,
                                        causal=causal, scale=s)
        sc = F_._block_scores_from_pooled(Q, K, block_size_m=bm, block_size_n=bn, scale=s)
        out.update({f"{name}.Q": np32(Q), f"{name}.K": np32(K), f"{name}.V": np32(V),
                    f"{name}.idx": idx.numpy().astype(np.int32), f"{name}.scores": np32(sc)})
        # indices from caller-supplied scores (unpadded offset rule)
        nq, nk = sc.shape[-2:]
        g = torch.Generator().manual_seed(5)
        bs = torch.randn(B, H, nq, nk, generator=g)
        idx2 = _topk_indices_from_scores(bs, k, nq, nk, bm, bn, Tq, Tk, causal, torch.device("cpu"))
        out.update({f"{name}.bs": np32(bs), f"{name}.idx_bs": idx2.numpy().astype(np.int32)})
        meta.append((name, dict(B=B, H=H, Tq=Tq, Tk=Tk, D=D, bm=bm, bn=bn, k=k, causal=causal,
                                dtype=str(dt))))

    # ---- selected forward + backward with fixed (canonical) indices ---------
    for name, (B, H, Tq, Tk, D, bm, bn, k, causal, dt) in {
        "sel_a": (1, 2, 256, 256, 32, 64, 64, 3, True, torch.bfloat16),
        "sel_b": (1, 2, 100, 200, 32, 32, 32, 4, True, torch.bfloat16),      # ragged
        "sel_c": (1, 2, 128, 192, 32, 64, 64, 2, False, torch.float32),
    }.items():
        Q, K, V, g = qkv(37, B, H, Tq, Tk, D, dt)
        dO = torch.randn(B, H, Tq, D, generator=g)
        idx = O.select_blocks(Q, K, block_size_m=bm, block_size_n=bn, top_k=k, causal=causal)
        Qd, Kd, Vd = (t.float().requires_grad_(True) for t in (Q, K, V))
        o, l = R.selected_attention_reference(Qd, Kd, Vd, block_size_n=bn, block_size_m=bm,
                                              top_k=k, block_indices=idx, causal=causal)
        on = torch.nan_to_num(o, nan=0.0, posinf=0.0, neginf=0.0)
        dQ, dK, dV = torch.autograd.grad(on, (Qd, Kd, Vd), grad_outputs=dO)
        out.update({f"{name}.Q": np32(Q), f"{name}.K": np32(K), f"{name}.V": np32(V),
                    f"{name}.dO": np32(dO), f"{name}.idx": idx.numpy(),
                    f"{name}.out": np32(o), f"{name}.lse": np32(l),
                    f"{name}.dQ": np32(torch.nan_to_num(dQ)), f"{name}.dK": np32(torch.nan_to_num(dK)),
                    f"{name}.dV": np32(torch.nan_to_num(dV))})
        meta.append((name, dict(B=B, H=H, Tq=Tq, Tk=Tk, D=D, bm=bm, bn=bn, k=k, causal=causal,
                                dtype=str(dt))))

    # ---- sliding -------------------------------------------------------------
    for name, (B, H, Tq, Tk, D, W, causal, dt) in {
        "sld_a": (1, 2, 256, 256, 32, 64, True, torch.bfloat16),
        "sld_b": (1, 2, 100, 300, 32, 48, True, torch.float32),
        "sld_c": (1, 2, 128, 128, 32, 32, False, torch.bfloat16),
    }.items():
        Q, K, V, _ = qkv(41, B, H, Tq, Tk, D, dt)
        o, l = R.sliding_attention_reference(Q.float(), K.float(), V.float(), window_size=W,
                                             causal=causal)
        out.update({f"{name}.Q": np32(Q), f"{name}.K": np32(K), f"{name}.V": np32(V),
                    f"{name}.out": np32(o), f"{name}.lse": np32(l)})
        meta.append((name, dict(B=B, H=H, Tq=Tq, Tk=Tk, D=D, W=W, causal=causal, dtype=str(dt))))

    # ---- compressed / sliding gradients (the reference's own backward route: autograd through its
    #      plain-torch functions with nan_to_num, nsa/triton/forward.py:84-120) ---------------------
    for name, (B, H, Tq, Tk, D, kind, par, causal) in {
        "gcmp_a": (1, 2, 128, 128, 32, "cmp", 32, True),
        "gcmp_b": (1, 2, 96, 200, 32, "cmp", 64, True),
        "gsld_a": (1, 2, 128, 128, 32, "sld", 48, True),
        "gsld_b": (1, 2, 100, 300, 32, "sld", 64, False),
    }.items():
        Q, K, V, g = qkv(71, B, H, Tq, Tk, D, torch.bfloat16, 0.7)
        dO = torch.randn(B, H, Tq, D, generator=g)
        Qd, Kd, Vd = (t.float().requires_grad_(True) for t in (Q, K, V))
        if kind == "cmp":
            o, _ = R.compressed_attention_reference(Qd, Kd, Vd, block_size_c=par, causal=causal)
        else:
            o, _ = R.sliding_attention_reference(Qd, Kd, Vd, window_size=par, causal=causal)
        on = torch.nan_to_num(o, nan=0.0, posinf=0.0, neginf=0.0)
        dQ, dK, dV = (torch.nan_to_num(t) for t in torch.autograd.grad(on, (Qd, Kd, Vd), grad_outputs=dO))
        out.update({f"{name}.Q": np32(Q), f"{name}.K": np32(K), f"{name}.V": np32(V), f"{name}.dO": np32(dO),
                    f"{name}.dQ": np32(dQ), f"{name}.dK": np32(dK), f"{name}.dV": np32(dV)})
        meta.append((name, dict(B=B, H=H, Tq=Tq, Tk=Tk, D=D, kind=kind, par=par, causal=causal)))

    # ---- combined forward with gates -----------------------------------------
    for name, (B, H, T, D, act) in {
        "nsa_a": (1, 2, 256, 32, "sigmoid"),
        "nsa_b": (1, 2, 256, 32, "softmax"),
    }.items():
        Q, K, V, g = qkv(53, B, H, T, T, D, torch.bfloat16)
        gates = torch.randn(B, H, T, 3, generator=g)
        cfg = R.NSAConfig(block_size_c=32, block_size_n=32, block_size_m=32, top_k=3,
                          window_size=48, gate_activation=act)
        idx = O.select_blocks(Q, K, block_size_m=32, block_size_n=32, top_k=3, causal=True)
        # the reference's combined function scores in fp32 from its own inputs; feed the
        # canonical indices through block_scores so both sides gather the same blocks
        nq = nk = T // 32
        bs = torch.full((B, H, nq, nk), -1e9)
        bs.scatter_(-1, idx.long(), torch.arange(3, 0, -1.0).expand(B, H, nq, 3).contiguous())
        o = R.nsa_attention_reference(Q.float(), K.float(), V.float(), cfg, gates=gates,
                                      block_scores=bs)
        oc = GT.combine(Q, K, V, gates.to(torch.bfloat16), activation=act)   # bf16 rounding chain
        out.update({f"{name}.Q": np32(Q), f"{name}.K": np32(K), f"{name}.V": np32(V),
                    f"{name}.gates": np32(gates), f"{name}.idx": idx.numpy(),
                    f"{name}.out": np32(o), f"{name}.combine_bf16": np32(oc)})
        meta.append((name, dict(B=B, H=H, T=T, D=D, act=act)))

    # ---- fp8 quantise / dequantise ------------------------------------------
    for name, fmt in {"fp8_e4m3": torch.float8_e4m3fn, "fp8_e5m2": torch.float8_e5m2}.items():
        g = torch.Generator().manual_seed(61)
        x = torch.randn(4, 257, generator=g)
        x = torch.where(torch.rand(4, 257, generator=g) < 0.01, x * 20, x).to(torch.bfloat16)
        x8, sc = FP8.quantize_to_fp8(x, fmt=fmt)
        deq = x8.to(torch.bfloat16) * sc
        out.update({f"{name}.x": np32(x), f"{name}.bits": x8.view(torch.uint8).numpy(),
                    f"{name}.scale": np.array([sc], dtype=np.float64), f"{name}.deq": np32(deq)})
        meta.append((name, dict(fmt=str(fmt))))

    np.savez_compressed(os.path.join(HERE, "reference_golden.npz"), **out)
    with open(os.path.join(HERE, "reference_golden.meta.txt"), "w") as f:
        f.write(f"torch {torch.__version__}\n")
        for n, m in meta:
            f.write(f"{n}: {m}\n")
    print("wrote", len(out), "arrays")


if __name__ == "__main__":
    main()
