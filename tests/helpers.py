"""Seeded inputs and comparison helpers shared by the tests."""
import torch


def make_qkv(seed, B, H, Hkv, Tq, Tk, D, dtype=torch.bfloat16, amp=1.0):
    """Q, K, V ~ N(0,1)*amp from a CPU generator in the order Q, K, V (the reference's order)."""
    g = torch.Generator().manual_seed(seed)
    Q = (torch.randn(B, H, Tq, D, generator=g) * amp).to(dtype)
    K = (torch.randn(B, Hkv, Tk, D, generator=g) * amp).to(dtype)
    V = (torch.randn(B, Hkv, Tk, D, generator=g) * amp).to(dtype)
    return Q, K, V, g


def max_abs(a, ref, mask=None):
    d = (a.float().cpu() - ref.float().cpu()).abs()
    if mask is not None:
        d = d[mask]
    return float(d.max()) if d.numel() else 0.0


def check_out_lse(out, lse, ref_out, ref_lse, tol_out, tol_lse=1e-2):
    """Rows the oracle calls empty must be (0, -inf); the rest within tolerance."""
    ref_lse = ref_lse.cpu()
    lse = lse.float().cpu()
    empty = ref_lse == float("-inf")
    assert torch.equal(lse == float("-inf"), empty), "pattern of empty rows differs"
    assert float(out.float().cpu()[empty].abs().sum()) == 0.0
    fin = ~empty
    assert max_abs(lse, ref_lse, fin) <= tol_lse, max_abs(lse, ref_lse, fin)
    assert max_abs(out, ref_out, fin) <= tol_out, max_abs(out, ref_out, fin)
