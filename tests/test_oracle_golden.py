"""Pins the CPU oracle to the reference's own outputs (tests/golden/reference_golden.npz,
made by tests/golden/make_golden.py from the reference's plain-torch functions)."""
import numpy as np
import torch

from oracle import nsa_oracle as O

DT = {"torch.float32": torch.float32, "torch.bfloat16": torch.bfloat16, "torch.float16": torch.float16}


def T(g, key, dtype=torch.float32):
    return torch.from_numpy(np.asarray(g[key])).to(dtype)


def finite_close(a, ref, atol, rtol=0.0):
    ok = torch.isfinite(ref)
    assert ok.any()
    d = (a[ok] - ref[ok]).abs()
    assert bool((d <= atol + rtol * ref[ok].abs()).all()), float(d.max())


CMP = {"cmp_a": (32, True, "torch.float32"), "cmp_b": (64, True, "torch.bfloat16"),
       "cmp_c": (32, False, "torch.bfloat16")}


def test_compressed_matches_reference(golden):
    for name, (bc, causal, dt) in CMP.items():
        Q, K, V = (T(golden, f"{name}.{x}", DT[dt]) for x in "QKV")
        out, lse = O.compressed_attention(Q.float(), K.float(), V.float(), block_size_c=bc, causal=causal)
        ref_o, ref_l = T(golden, f"{name}.out"), T(golden, f"{name}.lse")
        finite_close(out, ref_o, 2e-5)
        finite_close(lse, ref_l, 2e-5)
        # rows the reference leaves undefined (NaN) are the rows the oracle reports empty
        empty = ~torch.isfinite(ref_l)
        assert torch.equal(empty, lse == float("-inf"))
        assert float(out[empty].abs().sum()) == 0.0
        # pooled keys: bit-identical for 16-bit inputs (one rounding of an fp32 sum);
        # for fp32 inputs only the summation order differs
        if DT[dt] == torch.float32:
            assert torch.allclose(O.pool_mean(K, bc), T(golden, f"{name}.Kc"), atol=1e-6)
        else:
            assert torch.equal(O.pool_mean(K, bc).float(), T(golden, f"{name}.Kc"))


IDX = {"sel_idx_a": (64, 64, 4, True, "torch.bfloat16"), "sel_idx_b": (32, 32, 5, True, "torch.bfloat16"),
       "sel_idx_c": (64, 64, 3, False, "torch.float16")}


def test_block_selection_matches_reference(golden):
    for name, (bm, bn, k, causal, dt) in IDX.items():
        Q, K = T(golden, f"{name}.Q", DT[dt]), T(golden, f"{name}.K", DT[dt])
        idx, masked = O.select_blocks(Q, K, block_size_m=bm, block_size_n=bn, top_k=k, causal=causal,
                                      return_scores=True)
        ref_idx = T(golden, f"{name}.idx", torch.int32)
        sc = O.block_scores(Q, K, block_size_m=bm, block_size_n=bn)
        assert torch.allclose(sc, T(golden, f"{name}.scores"), atol=1e-6, rtol=1e-6)
        # exact on every slot whose score is finite; -inf slots are filled lowest-index-first
        fin = torch.isfinite(torch.gather(masked, -1, idx.long()))
        assert torch.equal(idx[fin], ref_idx[fin])
        assert fin.float().mean() > 0.5
        # the canonical fill: ascending illegal ids
        nq = idx.shape[2]
        for q in range(nq):
            row, f = idx[0, 0, q], fin[0, 0, q]
            tail = row[~f]
            assert torch.equal(tail, torch.sort(tail).values)
        # caller-supplied scores (unpadded offset rule)
        bs = T(golden, f"{name}.bs")
        Tq, Tk = Q.shape[2], K.shape[2]
        idx2 = O.indices_from_scores(bs, top_k=k, block_size_m=bm, block_size_n=bn, Tq=Tq, Tk=Tk, causal=causal)
        ref2 = T(golden, f"{name}.idx_bs", torch.int32)
        nq, nk = bs.shape[-2:]
        legal = O.legal_blocks(nq, nk, bm, bn, Tk - Tq) if causal else torch.ones(nq, nk, dtype=torch.bool)
        fin2 = torch.gather(legal.expand(bs.shape), -1, idx2.long())
        assert torch.equal(idx2[fin2], ref2[fin2])


SEL = {"sel_a": (64, 64, True), "sel_b": (32, 32, True), "sel_c": (64, 64, False)}


def test_selected_forward_backward_match_reference(golden):
    for name, (bm, bn, causal) in SEL.items():
        Q, K, V, dO = (T(golden, f"{name}.{x}") for x in ("Q", "K", "V", "dO"))
        idx = T(golden, f"{name}.idx", torch.int32)
        out, lse = O.selected_attention(Q, K, V, idx, block_size_n=bn, block_size_m=bm, causal=causal)
        finite_close(out, T(golden, f"{name}.out"), 2e-5)
        finite_close(lse, T(golden, f"{name}.lse"), 2e-5)
        dQ, dK, dV = O.selected_backward(dO, Q, K, V, idx, block_size_n=bn, block_size_m=bm, causal=causal)
        for a, key in ((dQ, "dQ"), (dK, "dK"), (dV, "dV")):
            assert torch.allclose(a, T(golden, f"{name}.{key}"), atol=5e-5, rtol=1e-4), key


SLD = {"sld_a": (64, True), "sld_b": (48, True), "sld_c": (32, False)}


def test_sliding_matches_reference(golden):
    for name, (W, causal) in SLD.items():
        Q, K, V = (T(golden, f"{name}.{x}") for x in "QKV")
        out, lse = O.sliding_attention(Q, K, V, window_size=W, causal=causal)
        finite_close(out, T(golden, f"{name}.out"), 2e-5)
        finite_close(lse, T(golden, f"{name}.lse"), 2e-5)
        # a band of rows against the full key set gives the same rows
        o2, l2 = O.sliding_attention(Q, K, V, window_size=W, causal=causal, rows=(32, 96))
        assert torch.allclose(o2, out[:, :, 32:96], atol=1e-6)


GRAD = {"gcmp_a": ("cmp", dict(block_size_c=32, causal=True)), "gcmp_b": ("cmp", dict(block_size_c=64, causal=True)),
        "gsld_a": ("sld", dict(window_size=48, causal=True)), "gsld_b": ("sld", dict(window_size=64, causal=False))}


def test_compressed_and_sliding_gradients_match_reference(golden):
    for name, (kind, kw) in GRAD.items():
        Q, K, V, dO = (T(golden, f"{name}.{x}") for x in ("Q", "K", "V", "dO"))
        dQ, dK, dV = O.branch_backward(kind, dO, Q, K, V, **kw)
        for a, key in ((dQ, "dQ"), (dK, "dK"), (dV, "dV")):
            if name == "gcmp_a" and key == "dV":
                # This case has query rows without any visible pooled token.  The reference's route gives NaN
                # weights there, which its matmul backward spreads over EVERY pooled value before nan_to_num
                # zeroes them: its dV is identically 0.  The oracle (and the kernels) keep the gradient of
                # the rows that do have keys; only that it is finite and non-zero is checked here.
                assert float(T(golden, f"{name}.{key}").abs().max()) == 0.0
                assert torch.isfinite(a).all() and float(a.abs().max()) > 0
                continue
            assert torch.allclose(a, T(golden, f"{name}.{key}"), atol=5e-5, rtol=1e-4), (name, key)


def test_combined_forward_and_combine_match_reference(golden):
    for name, act in (("nsa_a", "sigmoid"), ("nsa_b", "softmax")):
        Q, K, V, gates = (T(golden, f"{name}.{x}") for x in ("Q", "K", "V", "gates"))
        idx = T(golden, f"{name}.idx", torch.int32)
        out = O.nsa_forward(Q, K, V, block_size_c=32, block_size_n=32, block_size_m=32, top_k=3,
                            window_size=48, gate_logits=gates, gate_activation=act, block_indices=idx)
        finite_close(out, T(golden, f"{name}.out"), 3e-5)
        band = O.nsa_forward(Q, K, V, block_size_c=32, block_size_n=32, block_size_m=32, top_k=3,
                             window_size=48, gate_logits=gates, gate_activation=act, block_indices=idx,
                             rows=(64, 160))
        assert torch.allclose(band, out[:, :, 64:160], atol=1e-6)
        bq, bk, bv = (x.to(torch.bfloat16) for x in (Q, K, V))
        oc = O.combine(bq, bk, bv, gates.to(torch.bfloat16), activation=act)
        assert torch.equal(oc.float(), T(golden, f"{name}.combine_bf16"))


def test_fp8_quantise_matches_reference(golden):
    for name, fmt in (("fp8_e4m3", torch.float8_e4m3fn), ("fp8_e5m2", torch.float8_e5m2)):
        x = T(golden, f"{name}.x", torch.bfloat16)
        x8, sc = O.quantize_to_fp8(x, fmt=fmt)
        assert sc == float(golden[f"{name}.scale"][0])
        assert np.array_equal(x8.view(torch.uint8).numpy(), golden[f"{name}.bits"])
        assert torch.equal(O.dequantize_fp8(x8, sc).float(), T(golden, f"{name}.deq"))


def test_unpinned_extensions_collapse_to_pinned_cases(golden):
    """GQA with one group, stride == block and zero forced blocks are the pinned paths."""
    name = "sel_a"
    Q, K, V = (T(golden, f"{name}.{x}") for x in "QKV")
    idx = T(golden, f"{name}.idx", torch.int32)
    # GQA: a shared KV head equals the reference run on repeated heads
    K1, V1 = K[:, :1], V[:, :1]
    o_g, _ = O.selected_attention(Q, K1, V1, idx, causal=True)
    o_r, _ = O.selected_attention(Q, K1.repeat(1, 2, 1, 1), V1.repeat(1, 2, 1, 1), idx, causal=True)
    assert torch.equal(o_g, o_r)
    # group-shared indices == the same index rows repeated per head
    o_s, _ = O.selected_attention(Q, K1, V1, idx[:, :1], causal=True)
    o_p, _ = O.selected_attention(Q, K1, V1, idx[:, :1].repeat(1, 2, 1, 1), causal=True)
    assert torch.equal(o_s, o_p)
    # stride == block is the reference pooling
    assert torch.equal(O.pool_mean(K, 32, 32), O.pool_mean(K, 32))
    # overlapping windows: window c of (block 32, stride 16) is rows [16c, 16c+32)
    p = O.pool_mean(K, 32, 16)
    assert p.shape[2] == (K.shape[2] - 32) // 16 + 1
    assert torch.allclose(p[:, :, 3], K[:, :, 48:80].mean(2), atol=1e-6)
    # forced blocks: 0 forced == plain; forced blocks come first and are legal
    a = O.select_blocks(Q, K, top_k=3)
    b = O.select_blocks(Q, K, top_k=3, force_first=0, force_local=0)
    assert torch.equal(a, b)
    f = O.select_blocks(Q, K, top_k=3, force_first=1, force_local=2)
    nq = f.shape[2]
    for q in range(2, nq):
        assert set(f[0, 0, q].tolist()) == {0, q - 1, q} if q >= 2 else True


LAYER = {"layer_a": dict(n_heads=4, head_dim=64, block_size_c=32, top_k=8, window_size=96, gate_activation="sigmoid"),
         "layer_b": dict(n_heads=2, head_dim=128, block_size_c=64, top_k=4, window_size=64, gate_activation="softmax")}


def test_layer_oracle_matches_reference_module(layer_golden):
    """The caller of the forward (projections, rotary embedding, gate logits, transposes, output
    projection) against the reference's own module run on CPU (tests/golden/layer_golden.npz)."""
    g = layer_golden
    qr = O.rope(T(g, "layer_a.q_bthd").transpose(1, 2), T(g, "layer_a.cos"), T(g, "layer_a.sin"))
    assert torch.allclose(qr, T(g, "layer_a.q_rope"), atol=1e-6)
    for name, kw in LAYER.items():
        w = {k[len(name) + 3:]: T(g, k) for k in g.files if k.startswith(f"{name}.w.")}
        y = O.attention_layer(T(g, f"{name}.x"), w, T(g, f"{name}.cos"), T(g, f"{name}.sin"), **kw)
        ref = T(g, f"{name}.y")
        # tokens before the first complete compression block have no pooled key: the reference's fp32 route
        # gives NaN there (the kernels' convention is a zero compressed branch), every other token is compared
        ok = torch.isfinite(ref).all(-1)
        assert torch.equal(ok[0], torch.arange(ref.shape[1]) >= kw["block_size_c"] - 1)
        assert float((y - ref)[ok].abs().max()) <= 2e-5, float((y - ref)[ok].abs().max())


def test_compressed_probability_scorer_degenerate_cases():
    """The probability-based scorer has no counterpart in the reference (parity unpinned); its restatement is
    tied to pinned behaviour through cases that collapse onto it: every query row hands out exactly its
    softmax mass (1, or 0 without a visible compressed token), and with compression block = stride = selection
    block the score of a block is the compressed branch's own probability of that block's single token."""
    g = torch.Generator().manual_seed(7)
    Q = torch.randn(1, 4, 256, 32, generator=g).to(torch.bfloat16)
    K = torch.randn(1, 2, 256, 32, generator=g).to(torch.bfloat16)
    V = torch.zeros(1, 2, 256, 32)
    V[..., :4] = torch.eye(4).repeat_interleave(64, 0)            # row r carries one-hot(block of r) in its first 4 columns
    for bc, stride in ((32, 16), (32, 32), (64, 64)):
        sc = O.compressed_block_scores(Q, K, block_size_c=bc, stride_c=stride)
        rows_with_token = (torch.arange(256) >= bc - 1).view(4, 64).sum(1).float()      # per query block
        assert torch.allclose(sc.sum(-1), rows_with_token.expand(1, 4, 4), atol=1e-4)
        assert float(O.overlap_weights(O.n_pooled(256, bc, stride), 4, bc, stride, 64).sum(1).sub(1).abs().max()) == 0.0
        gs = O.compressed_block_scores(Q, K, block_size_c=bc, stride_c=stride, group_shared=True)
        assert torch.allclose(gs, sc.view(1, 2, 2, 4, 4).sum(2), atol=1e-5)
    # block = stride = 64: pooled token j IS selection block j, and attention over V = one-hot(block) returns the
    # per-row probabilities of the compressed branch
    sc = O.compressed_block_scores(Q, K, block_size_c=64, stride_c=64)
    probs = O.compressed_attention(Q, K, V, block_size_c=64)[0][..., :4]                  # [1,4,256,4]: p[i, block]
    assert torch.allclose(sc, probs.view(1, 4, 4, 64, 4).sum(3), atol=1e-5)


def test_learned_pooling_vs_reference():
    """pool="learned": the oracle against the reference's plain-torch compressed branch and combined forward
    (tests/golden/learned_pool_golden.npz, made by make_golden.py --part learned)."""
    import os
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "learned_pool_golden.npz"))
    T = lambda k: torch.from_numpy(np.asarray(g[k]))
    for name, bc in (("lp_a", 32), ("lp_b", 64)):
        o, l = O.compressed_attention(T(f"{name}.Q"), T(f"{name}.K"), T(f"{name}.V"), block_size_c=bc, causal=True,
                                      pool_proj_k=T(f"{name}.pk"), pool_proj_v=T(f"{name}.pv"))
        rl = T(f"{name}.lse")
        fin = torch.isfinite(rl)
        assert torch.equal(torch.isfinite(l), fin)
        assert float((o - torch.nan_to_num(T(f"{name}.out")))[fin].abs().max()) <= 1e-5
        assert float((l - rl)[fin].abs().max()) <= 1e-5
    ref = T("lp_nsa.out")
    idx = O.select_blocks(T("lp_nsa.Q"), T("lp_nsa.K"), block_size_m=32, block_size_n=32, top_k=3)
    out = O.nsa_forward(T("lp_nsa.Q"), T("lp_nsa.K"), T("lp_nsa.V"), block_size_c=32, block_size_n=32, block_size_m=32, top_k=3,
                        window_size=48, gate_logits=T("lp_nsa.gates"), block_indices=idx, pool_proj_k=T("lp_nsa.pk"),
                        pool_proj_v=T("lp_nsa.pv"))
    fin = torch.isfinite(ref).all(-1)
    assert float((out - ref)[fin].abs().max()) <= 1e-4


def test_moba_routing_vs_reference():
    """The oracle's MoBA routing against the reference's lists (tests/golden/moba_golden.npz): per query block the same
    SET of legal blocks; the same order too wherever every row has at least top_k_per_query legal blocks (below that
    the reference's top-k returns arbitrary illegal ids, which change its union's size and so its ordering rule)."""
    import os
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "moba_golden.npz"))
    for name in ("moba_a", "moba_b", "moba_c"):
        Q, K = (torch.from_numpy(np.asarray(g[f"{name}.{x}"])).to(torch.bfloat16) for x in "QK")
        ref = torch.from_numpy(np.asarray(g[f"{name}.idx"]))
        kq, cap, causal = (int(x) for x in g[f"{name}.par"])
        mine = O.moba_block_indices(Q, K, top_k_per_query=kq, top_k_cap=cap, causal=bool(causal))
        assert mine.shape == ref.shape
        nq, nk = ref.shape[2], (K.shape[2] + 63) // 64
        off = nk * 64 - nq * 64
        for h in range(ref.shape[1]):
            for qb in range(nq):
                lim = (qb * 64 + 63 + off) // 64 if causal else nk - 1
                a = [int(x) for x in ref[0, h, qb] if x <= lim and x < nk]
                b = [int(x) for x in mine[0, h, qb] if x < nk]
                assert set(a) == set(b), (name, h, qb, a, b)
                first_row_legal = (qb * 64 + off) // 64 + 1 if causal else nk
                if first_row_legal >= kq:
                    assert a == b, (name, h, qb, a, b)
