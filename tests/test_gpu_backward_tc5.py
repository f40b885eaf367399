"""Selected-branch backward on the tcgen05 engine (inverted block lists, dK/dV accumulated per key block in
tensor memory, dQ in a query-major pass; no floating-point atomics) against the fp32 oracle, against the
generic engine, and against itself (bit-repeatability).  Everything goes through the C ABI.
Tolerance: max-abs <= 2e-2 * max(1, max|reference|) for bf16/fp16 gradients."""
import ctypes as C

import pytest
import torch

from helpers import make_qkv, max_abs
from oracle import nsa_oracle as O

pytestmark = pytest.mark.gpu

TOL16 = 2e-2


@pytest.fixture(scope="module")
def nsa():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import nsa_from_scratch_b200 as pkg
    return pkg


def _run(nsa, engine, dO, Q, K, V, idx, causal=True, scale=None):
    from nsa_from_scratch_b200 import ops
    D = Q.shape[-1]
    scale = 1.0 / D ** 0.5 if scale is None else scale
    Qc, Kc, Vc, dOc, ic = (t.cuda() for t in (Q, K, V, dO, idx))
    out, lse = nsa.selected_attention(Qc, Kc, Vc, block_indices=ic, causal=causal, scale=scale)
    delta = ops.bwd_delta(dOc, out)
    ops.set_bwd_engine(engine)
    try:
        res = ops.selected_bwd(dOc, Qc, Kc, Vc, lse, delta, ic, bm=64, bn=64, causal=causal, scale=scale,
                               offset=K.shape[2] - Q.shape[2], dq_fp32=True)
        ops.device_status()
    finally:
        ops.set_bwd_engine("auto")
    return res


def _check(got, ref, what):
    for g, r, nm in zip(got, ref, ("dQ", "dK", "dV")):
        err, mag = max_abs(g, r), float(r.abs().max())
        assert err <= TOL16 * max(1.0, mag), (what, nm, err, mag)


# (B, H, Hkv, Tq, Tk, D, top_k, lists shared by the group, dtype)
CASES = [
    (1, 4, 4, 256, 256, 64, 3, False, torch.bfloat16),     # multi-head attention, one list per head (the reference's case)
    (1, 8, 2, 256, 256, 128, 4, False, torch.bfloat16),    # grouped heads, lists per head, D=128
    (2, 4, 1, 192, 192, 64, 3, True, torch.bfloat16),      # one list per KV head
    (1, 6, 2, 320, 320, 64, 4, True, torch.float16),       # odd number of head pairs per group (3 heads), fp16
    (1, 4, 2, 200, 456, 64, 5, True, torch.bfloat16),      # ragged lengths, queries aligned with the tail of the keys
    (1, 4, 2, 200, 456, 128, 5, False, torch.bfloat16),
    (1, 16, 1, 512, 512, 128, 8, True, torch.bfloat16),    # 16 heads share every list
]


@pytest.mark.parametrize("case", CASES)
def test_tc5_backward_vs_oracle_and_generic(nsa, case):
    B, H, Hkv, Tq, Tk, D, k, shared, dt = case
    Q, K, V, g = make_qkv(21, B, H, Hkv, Tq, Tk, D, dtype=dt)
    dO = torch.randn(B, H, Tq, D, generator=g).to(dt)
    idx = O.select_blocks(Q, K, top_k=k, causal=True, force_first=1, force_local=2, group_shared=shared)
    assert idx.shape[1] == (Hkv if shared else H)
    ref = O.selected_backward(dO, Q, K, V, idx, causal=True)
    got = _run(nsa, "tcgen05", dO, Q, K, V, idx)
    _check(got, ref, "tcgen05 vs oracle")
    gen = _run(nsa, "generic", dO, Q, K, V, idx)
    _check(got, [t.cpu() for t in gen], "tcgen05 vs generic")
    # no atomics on floating-point data: a second run gives the same bits
    again = _run(nsa, "tcgen05", dO, Q, K, V, idx)
    for a_, b_ in zip(got, again):
        assert torch.equal(a_, b_)


def test_tc5_backward_duplicates_sentinel_noncausal(nsa):
    """A block listed twice counts twice, ids outside [0, nk) are skipped, without the causal rule."""
    B, H, Hkv, T, D = 1, 4, 2, 256, 64
    Q, K, V, g = make_qkv(22, B, H, Hkv, T, T, D)
    dO = torch.randn(B, H, T, D, generator=g).to(torch.bfloat16)
    nk = T // 64
    for Hi in (H, Hkv):
        idx = torch.tensor([0, 0, nk, 2, -1, 1], dtype=torch.int32).expand(B, Hi, nk, 6).contiguous()
        for causal in (False, True):
            ref = O.selected_backward(dO, Q, K, V, idx, causal=causal)
            got = _run(nsa, "tcgen05", dO, Q, K, V, idx, causal=causal)
            _check(got, ref, f"Hi={Hi} causal={causal}")


def test_tc5_backward_long_lists_split_into_segments(nsa):
    """Every query block lists block 0, so its list (all query blocks x all heads of the group = 4*48 row groups)
    is longer than one work item takes: the partial dK/dV of the segments are summed by the reduce kernel."""
    B, H, Hkv, T, D = 1, 4, 1, 64 * 48, 64
    Q, K, V, g = make_qkv(23, B, H, Hkv, T, T, D)
    dO = torch.randn(B, H, T, D, generator=g).to(torch.bfloat16)
    for shared in (True, False):
        idx = O.select_blocks(Q, K, top_k=4, causal=True, force_first=1, force_local=2, group_shared=shared)
        ref = O.selected_backward(dO, Q, K, V, idx, causal=True)
        got = _run(nsa, "tcgen05", dO, Q, K, V, idx)
        _check(got, ref, f"shared={shared}")
        again = _run(nsa, "tcgen05", dO, Q, K, V, idx)
        for a_, b_ in zip(got, again):
            assert torch.equal(a_, b_)


def test_tc5_backward_accumulates_into_dk_dv_and_bf16_dq(nsa):
    """dK_f / dV_f are added to (the caller's zeroing contract); dQ may be asked for in the 16-bit type."""
    from nsa_from_scratch_b200 import _lib as L, ops
    B, H, Hkv, T, D = 1, 4, 2, 256, 64
    Q, K, V, g = make_qkv(24, B, H, Hkv, T, T, D)
    dO = torch.randn(B, H, T, D, generator=g).to(torch.bfloat16)
    idx = O.select_blocks(Q, K, top_k=3, causal=True, group_shared=True)
    base = _run(nsa, "tcgen05", dO, Q, K, V, idx)
    Qc, Kc, Vc, dOc, ic = (t.cuda() for t in (Q, K, V, dO, idx))
    out, lse = nsa.selected_attention(Qc, Kc, Vc, block_indices=ic)
    delta = ops.bwd_delta(dOc, out)
    dQ = torch.empty(B, H, T, D, device="cuda", dtype=torch.bfloat16)
    dK = torch.full((B, Hkv, T, D), 1.5, device="cuda", dtype=torch.float32)
    dV = torch.full((B, Hkv, T, D), -2.0, device="cuda", dtype=torch.float32)
    a = L.BwdArgs()
    a.Q, a.K, a.V, a.dO = Qc.data_ptr(), Kc.data_ptr(), Vc.data_ptr(), dOc.data_ptr()
    a.lse, a.delta, a.idx = lse.data_ptr(), delta.data_ptr(), ic.data_ptr()
    a.dQ, a.dK_f, a.dV_f = dQ.data_ptr(), dK.data_ptr(), dV.data_ptr()
    a.B, a.H, a.Hkv, a.Hi, a.Tq, a.Tk, a.D = B, H, Hkv, Hkv, T, T, D
    a.nq, a.top_k, a.bm, a.bn, a.sel_key_limit = T // 64, idx.shape[3], 64, 64, T
    a.offset, a.causal, a.dtype, a.dq_dtype, a.scale = 0, 1, L.BF16, L.BF16, 1.0 / D ** 0.5
    a.branch, a.engine = L.BRANCH_SELECTED, L.ENGINE_TCGEN05
    lib = L.load()
    need = int(lib.nsa_attention_bwd_scratch_bytes(C.byref(a)))
    assert need > 0
    # the tcgen05 engine without scratch is an argument error, reported on the host before any launch
    assert lib.nsa_attention_bwd(C.byref(a), L.stream_ptr()) == -1
    assert b"scratch" in lib.nsa_last_error()
    scratch = torch.empty(need, device="cuda", dtype=torch.uint8)
    a.scratch, a.scratch_bytes = scratch.data_ptr(), need
    L.check(lib.nsa_attention_bwd(C.byref(a), L.stream_ptr()), "nsa_attention_bwd")
    ops.device_status()
    assert torch.equal(dK - 1.5, (base[1] + 1.5) - 1.5)
    assert torch.equal(dV + 2.0, (base[2] - 2.0) + 2.0)
    assert torch.equal(dQ, base[0].to(torch.bfloat16))
    # shapes the engine does not take report 0 bytes (the generic engine runs them)
    a.bm = a.bn = 32
    assert int(lib.nsa_attention_bwd_scratch_bytes(C.byref(a))) == 0
