"""The kernels driven through the reference's own module names.

`compat.install()` makes `nsa.triton.compressed|selected|sliding|gating|forward|backward|fp8` and `nsa.cuda`
resolve to this package.  The cases below repeat the shapes, dtypes, input generators (device generator seeded
as the reference's tests seed it) and tolerances of the reference's acceptance tests, import every function by
the reference's name, and compare with the CPU oracle (the reference's plain-torch functions are not on the GPU
box; the oracle is pinned to them by the golden fixtures).  Cited per test: the reference test it mirrors.

When a checkout of the reference is importable (environment variable NSA_REFERENCE_CHECKOUT), its own tests/
directory is additionally run in a subprocess with the shim installed first."""
import os
import subprocess
import sys

import pytest
import torch

from oracle import nsa_oracle as O

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def shim():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    keep = {k: v for k, v in sys.modules.items() if k == "nsa" or k.startswith("nsa.")}
    for k in keep:
        del sys.modules[k]
    from nsa_from_scratch_b200 import compat
    compat.install()
    yield
    for k in [k for k in sys.modules if k == "nsa" or k.startswith("nsa.")]:
        del sys.modules[k]
    sys.modules.update(keep)


def _qkv(B, H, Tq, Tk, D, dtype, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    Q = torch.randn(B, H, Tq, D, dtype=dtype, device="cuda", generator=g)
    K = torch.randn(B, H, Tk, D, dtype=dtype, device="cuda", generator=g)
    V = torch.randn(B, H, Tk, D, dtype=dtype, device="cuda", generator=g)
    return Q, K, V, g


def _allclose(got, ref, rtol, atol, mask=None):
    d = (got.float().cpu() - ref.float().cpu()).abs()
    bound = atol + rtol * ref.float().cpu().abs()
    bad = d > bound
    if mask is not None:
        bad = bad & mask
    assert int(bad.sum()) == 0, (int(bad.sum()), float(d[bad].max()))


# tests/test_compressed_forward.py:25-31,109-135: out within 1e-2 relative + 1e-2 absolute, lse within 1e-2
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("shape", [(1, 4, 128, 128, 64), (2, 8, 256, 256, 64), (1, 4, 512, 1024, 64)])
def test_compressed_by_reference_name(shim, shape, dtype, causal):
    from nsa.triton.compressed import compressed_attention
    B, H, Tq, Tk, D = shape
    Q, K, V, _ = _qkv(B, H, Tq, Tk, D, dtype, 0)
    out, lse = compressed_attention(Q, K, V, block_size_c=64, causal=causal)
    assert out.dtype == dtype and lse.dtype == torch.float32
    ro, rl = O.compressed_attention(Q.cpu(), K.cpu(), V.cpu(), block_size_c=64, causal=causal)
    fin = torch.isfinite(rl)
    assert torch.equal(torch.isfinite(lse.cpu()), fin)
    _allclose(out, ro, 1e-2, 1e-2, fin.unsqueeze(-1).expand_as(ro))
    assert float((lse.cpu() - rl)[fin].abs().max()) < 1e-2


# tests/test_selected_forward.py:141-193: scores -> shared top-k indices, max relative error < 1e-2 (fp16/bf16)
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape", [(1, 4, 128, 128, 64, 2, 32, 32), (1, 8, 1024, 2048, 64, 8, 64, 64), (2, 8, 512, 1024, 64, 4, 64, 64)])
def test_selected_by_reference_name(shim, shape, dtype):
    from nsa.triton.selected import selected_attention, _topk_indices_from_scores
    B, H, Tq, Tk, D, k, bm, bn = shape
    Q, K, V, _ = _qkv(B, H, Tq, Tk, D, dtype, 0)
    g = torch.Generator(device="cuda").manual_seed(1)
    scores = torch.randn(B, H, (Tq + bm - 1) // bm, (Tk + bn - 1) // bn, dtype=torch.float32, device="cuda", generator=g)
    nq, nk = (Tq + bm - 1) // bm, (Tk + bn - 1) // bn
    idx = _topk_indices_from_scores(scores, top_k=k, n_q_blocks=nq, n_kv_blocks=nk, block_size_m=bm, block_size_n=bn,
                                    Tq=Tq, Tk=Tk, causal=True)
    ref_idx = O.indices_from_scores(scores.cpu(), top_k=k, block_size_m=bm, block_size_n=bn, Tq=Tq, Tk=Tk, causal=True)
    assert torch.equal(idx.cpu(), ref_idx)
    out, lse = selected_attention(Q, K, V, block_size_n=bn, block_size_m=bm, top_k=k, block_scores=scores, causal=True)
    out2, _ = selected_attention(Q, K, V, block_size_n=bn, block_size_m=bm, top_k=k, block_indices=idx, causal=True,
                                 num_warps=8, num_stages=3)
    assert torch.equal(out, out2)
    ro, rl = O.selected_attention(Q.cpu(), K.cpu(), V.cpu(), ref_idx, block_size_n=bn, block_size_m=bm, causal=True)
    fin = torch.isfinite(rl)
    rel = float((out.float().cpu() - ro)[fin].abs().max() / (ro[fin].abs().max() + 1e-6))
    assert rel < 1e-2, rel
    assert float((lse.cpu() - rl)[fin].abs().max()) < 1e-2


# tests/test_selected_forward.py:196-227: every block selected == full causal attention
def test_selected_all_blocks_is_full_attention(shim):
    from nsa.triton.selected import selected_attention
    B, H, T, D = 1, 4, 256, 64
    Q, K, V, _ = _qkv(B, H, T, T, D, torch.bfloat16, 0)
    nk = T // 64
    idx = torch.arange(nk, device="cuda", dtype=torch.int32).expand(B, H, nk, nk).contiguous()
    out, _ = selected_attention(Q, K, V, top_k=nk, block_indices=idx, causal=True)
    ro, _ = O.sliding_attention(Q.cpu(), K.cpu(), V.cpu(), window_size=T, causal=True)
    assert float((out.float().cpu() - ro).abs().max()) < 2e-2


# tests/test_sliding_forward.py:40-84: relative error < 1e-2, lse < 1e-2; :86-103 window >= Tk == full attention
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("shape", [(1, 4, 128, 128, 64), (2, 8, 256, 256, 64), (1, 4, 1024, 1024, 64)])
def test_sliding_by_reference_name(shim, shape, dtype, causal):
    from nsa.triton.sliding import sliding_attention
    B, H, Tq, Tk, D = shape
    Q, K, V, _ = _qkv(B, H, Tq, Tk, D, dtype, 0)
    out, lse = sliding_attention(Q, K, V, window_size=64, causal=causal)
    ro, rl = O.sliding_attention(Q.cpu(), K.cpu(), V.cpu(), window_size=64, causal=causal)
    rel = float((out.float().cpu() - ro).abs().max() / (ro.abs().max() + 1e-6))
    assert rel < 1e-2, rel
    assert float((lse.cpu() - rl).abs().max()) < 1e-2


# tests/test_combined_forward.py:20-68: nsa_forward vs the plain-torch forward, rtol 1e-2 / atol 2e-2; :71-108 softmax gates
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("act", ["sigmoid", "softmax"])
@pytest.mark.parametrize("shape", [(1, 4, 128, 128, 64), (2, 4, 256, 256, 64), (1, 8, 512, 1024, 64)])
def test_combined_by_reference_name(shim, shape, dtype, act):
    from nsa.reference import NSAConfig
    from nsa.triton.forward import nsa_forward, _resolve_block_indices
    B, H, Tq, Tk, D = shape
    cfg = NSAConfig(block_size_c=32, block_size_n=32, block_size_m=32, top_k=4, window_size=64, causal=True,
                    gate_activation=act)
    Q, K, V, g = _qkv(B, H, Tq, Tk, D, dtype, 0)
    gates = torch.randn(B, H, Tq, 3, device="cuda", dtype=dtype, generator=g)
    out = nsa_forward(Q, K, V, cfg, gate_logits=gates)
    assert out.shape == (B, H, Tq, D) and out.dtype == dtype
    idx = _resolve_block_indices(Q, K, block_size_m=32, block_size_n=32, top_k=4, causal=True, scale=D ** -0.5)
    ref_idx = O.select_blocks(Q.cpu(), K.cpu(), block_size_m=32, block_size_n=32, top_k=4)
    assert torch.equal(idx.cpu(), ref_idx)
    ref = O.nsa_forward(Q.cpu(), K.cpu(), V.cpu(), block_size_c=32, block_size_n=32, block_size_m=32, top_k=4,
                        window_size=64, gate_logits=gates.cpu(), gate_activation=act, block_indices=ref_idx)
    fin = torch.isfinite(ref).all(-1, keepdim=True).expand_as(ref)
    _allclose(out, torch.nan_to_num(ref), 1e-2, 2e-2, fin)


# tests/test_selected_backward.py:73-127: the autograd Function, gradients at rtol 1e-2 / atol 5e-2
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_selected_backward_by_reference_name(shim, dtype):
    from nsa.triton.forward import _SelectedFn, _resolve_block_indices
    from nsa.triton.backward import selected_backward
    B, H, Tq, Tk, D, k = 1, 4, 128, 256, 64, 4
    Q, K, V, g = _qkv(B, H, Tq, Tk, D, dtype, 1)
    idx = _resolve_block_indices(Q, K, block_size_m=64, block_size_n=64, top_k=k, causal=True, scale=D ** -0.5)
    Qt, Kt, Vt = (t.detach().clone().requires_grad_(True) for t in (Q, K, V))
    out = _SelectedFn.apply(Qt, Kt, Vt, 64, 64, k, idx, True, None)
    dO = torch.randn(out.shape, device="cuda", dtype=dtype, generator=g)
    out.backward(dO)
    rQ, rK, rV = O.selected_backward(dO.cpu(), Q.cpu(), K.cpu(), V.cpu(), idx.cpu(), causal=True)
    for got, ref in ((Qt.grad, rQ), (Kt.grad, rK), (Vt.grad, rV)):
        assert got.dtype == dtype
        _allclose(got, ref, 1e-2, 5e-2)
    # the functional entry point with the reference's keyword list
    from nsa.triton.selected import selected_attention
    o2, l2 = selected_attention(Q, K, V, top_k=k, block_indices=idx, causal=True)
    dQ, dK, dV = selected_backward(dO, Q, K, V, o2, l2, idx, block_size_m=64, block_size_n=64, causal=True,
                                   scale=D ** -0.5, Tq=Tq, Tk=Tk)
    for got, ref in ((dQ, rQ), (dK, rK), (dV, rV)):
        _allclose(got, ref, 1e-2, 5e-2)


# tests/test_fp8.py:20-75: quantise per tensor, fp8 selected attention vs the fp32 reference at rtol/atol 1e-1
@pytest.mark.parametrize("fmt", [torch.float8_e4m3fn, torch.float8_e5m2])
def test_fp8_by_reference_name(shim, fmt):
    from nsa.triton.fp8 import quantize_to_fp8, selected_attention_fp8
    from nsa.triton.forward import _resolve_block_indices
    B, H, Tq, Tk, D, k = 1, 4, 256, 512, 64, 4
    Q, K, V, _ = _qkv(B, H, Tq, Tk, D, torch.float32, 0)
    Q8, sQ = quantize_to_fp8(Q, fmt=fmt)
    K8, sK = quantize_to_fp8(K, fmt=fmt)
    V8, sV = quantize_to_fp8(V, fmt=fmt)
    assert Q8.dtype == fmt and isinstance(sQ, float)
    idx = _resolve_block_indices(Q.to(torch.bfloat16), K.to(torch.bfloat16), block_size_m=64, block_size_n=64, top_k=k,
                                 causal=True, scale=D ** -0.5)
    out, _ = selected_attention_fp8(Q8, K8, V8, sQ, sK, sV, block_size_n=64, block_size_m=64, top_k=k, block_indices=idx,
                                    causal=True)
    ro, rl = O.selected_attention(Q.cpu(), K.cpu(), V.cpu(), idx.cpu(), causal=True)
    fin = torch.isfinite(rl).unsqueeze(-1).expand_as(ro)
    _allclose(out, ro, 1e-1, 1e-1, fin)


# tests/test_cuda_selected.py:87-262 and tests/test_cuda_selected_bwd.py:114-117: the native-extension names
def test_native_extension_names(shim):
    import nsa.cuda as native
    ext = native._get_ext()
    assert hasattr(ext, "selected_attention_fwd_cuda") and hasattr(ext, "selected_attention_bwd_cuda")
    B, H, T, D, k = 1, 4, 256, 128, 2
    Q, K, V, g = _qkv(B, H, T, T, D, torch.bfloat16, 0)
    idx = O.select_blocks(Q.cpu(), K.cpu(), top_k=k).cuda()
    out, lse = native.selected_attention_cuda(Q, K, V, idx, 64, 64, k, True, D ** -0.5)
    ro, rl = O.selected_attention(Q.cpu(), K.cpu(), V.cpu(), idx.cpu(), causal=True)
    assert float((out.float().cpu() - ro).abs().max()) < 2e-2 and float((lse.cpu() - rl).abs().max()) < 1e-2
    dO = torch.randn(out.shape, device="cuda", dtype=torch.bfloat16, generator=g)
    dQ, dK, dV = native.selected_backward_cuda(dO, Q, K, V, out, lse, idx, 64, 64, k, True, D ** -0.5)
    rQ, rK, rV = O.selected_backward(dO.cpu(), Q.cpu(), K.cpu(), V.cpu(), idx.cpu(), causal=True)
    for got, ref in ((dQ, rQ), (dK, rK), (dV, rV)):
        _allclose(got, ref, 1e-2, 5e-2)


def test_reference_checkout_test_suite_through_the_shim():
    """With NSA_REFERENCE_CHECKOUT pointing at a checkout of the reference, its own kernel tests run against these
    kernels (MoBA routing, the fp64 gradcheck route and the strict-xfail case of its broken native backward are
    deselected; they exercise code outside this package).  Skipped when no checkout is configured."""
    ref = os.environ.get("NSA_REFERENCE_CHECKOUT")
    if not ref or not os.path.isdir(os.path.join(ref, "tests")):
        pytest.skip("NSA_REFERENCE_CHECKOUT is not set to a checkout of the reference")
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    boot = ("import sys; sys.path.insert(0, %r); sys.path.insert(0, %r); "
            "from nsa_from_scratch_b200 import compat; compat.install(); import pytest; "
            "sys.exit(pytest.main(['-q', '-x', %r, '--deselect', 'tests/test_moba.py', '-k', "
            "'not gradcheck and not moba and not training_step and not native_matches_triton']))") % (ref, ROOT, os.path.join(ref, "tests"))
    r = subprocess.run([sys.executable, "-c", boot], cwd=ref, capture_output=True, text=True, timeout=1800)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]
