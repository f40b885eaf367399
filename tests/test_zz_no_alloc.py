"""The allocation-free compressed-branch entry point (nsa_compressed_attention_static).

Some hosts cannot give the library scratch memory at call time: their device memory is planned
and handed out before start-up, or the call sits where cudaMalloc is not allowed.  For them the
pooled K/V live in an array inside the library.  This test drives that entry point through the
C ABI twice in a row (different inputs, so leftovers of the first call would show) and compares
with the ordinary two-step path (nsa_pool_mean + nsa_attention_fwd), then checks that a problem
too large for the built-in array is refused with a message.  It runs last on purpose."""
import ctypes as C

import pytest
import torch

from helpers import make_qkv, max_abs

pytestmark = pytest.mark.gpu


def test_static_scratch_entry_point_matches_regular_path_twice():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from nsa_from_scratch_b200 import _lib as L, ops
    lib = L.load()
    for seed, (B, H, Hkv, Tq, Tk, D, bc, st, causal) in enumerate([(1, 8, 2, 512, 512, 128, 32, 16, True),
                                                                  (2, 4, 4, 200, 456, 64, 64, 64, True)]):
        Q, K, V, _ = make_qkv(20 + seed, B, H, Hkv, Tq, Tk, D)
        Q, K, V = Q.cuda(), K.cuda(), V.cuda()
        scale = D ** -0.5
        out = torch.empty_like(Q)
        lse = torch.empty((B, H, Tq), device="cuda", dtype=torch.float32)
        rc = lib.nsa_compressed_attention_static(Q.data_ptr(), K.data_ptr(), V.data_ptr(), out.data_ptr(), lse.data_ptr(),
                                                 B, H, Hkv, Tq, Tk, D, bc, st, int(causal), C.c_float(scale), L.BF16,
                                                 L.stream_ptr())
        assert rc == 0, lib.nsa_last_error().decode()
        Kc, Vc = ops.pool_mean(K, bc, st), ops.pool_mean(V, bc, st)
        Tk_pad = Kc.shape[2] * bc if st == bc else Tk
        ref_out, ref_lse = ops.attention_fwd(Q, K, V, branches=L.BRANCH_COMPRESSED, fused=False, causal=causal, scale=scale,
                                             Kc=Kc, Vc=Vc, cmp_block=bc, cmp_stride=st, cmp_offset=Tk_pad - Tq)
        torch.cuda.synchronize()
        assert max_abs(out, ref_out) <= 2e-2
        fin = torch.isfinite(ref_lse.cpu())
        assert torch.equal(torch.isfinite(lse.cpu()), fin)
        assert max_abs(lse, ref_lse, fin) <= 1e-2
    ops.device_status()
    # beyond the built-in array: refused before anything is launched
    big = lib.nsa_compressed_attention_static(Q.data_ptr(), K.data_ptr(), V.data_ptr(), out.data_ptr(), None, 64, 64, 64,
                                              64, 1 << 20, 128, 32, 16, 1, C.c_float(0.1), L.BF16, L.stream_ptr())
    assert big == -2
    assert b"scratch" in lib.nsa_last_error()
