"""Head-parallel layout on one GPU: the ranks of a split are played one after the other in this process (the
all-gather of the block means is replaced by the concatenation it returns), and the pieces must equal the
unsplit forward: block indices bit for bit always, outputs bit for bit when a rank holds a multiple of four query
heads of a KV head (the benchmark shape on 8 GPUs holds 8).  The collective itself is covered by the two-rank gloo
test on CPU (tests/test_parallel_cpu.py)."""
import pytest
import torch

from helpers import make_qkv

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("shared", [True, False])
@pytest.mark.parametrize("world", [2, 4, 8])
def test_head_parallel_pieces_equal_the_unsplit_forward(world, shared, monkeypatch):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import nsa_from_scratch_b200 as nsa
    from nsa_from_scratch_b200 import forward as F, ops, parallel as P
    B, H, Hkv, T, D = 1, 16, 2, 1024, 128
    Q, K, V, g = make_qkv(41, B, H, Hkv, T, T, D)
    gates = torch.randn(B, H, T, 3, generator=g).to(torch.bfloat16)
    Q, K, V, gates = Q.cuda(), K.cuda(), V.cuda(), gates.cuda()
    cfg = nsa.NSAConfig(block_size_c=32, stride_c=16, top_k=6, window_size=128, force_first=1, force_local=2,
                        select_per_group=shared)
    ref = nsa.nsa_forward(Q, K, V, cfg, gate_logits=gates)
    ref_idx = F._resolve_block_indices(Q, K, block_size_m=64, block_size_n=64, top_k=6, causal=True, scale=D ** -0.5,
                                       force_first=1, force_local=2, shared_per_group=shared)
    parts = [P.head_partition(B, H, Hkv, world, r) for r in range(world)]
    shards = [P.shard_heads(Q, K, V, p, gates) for p in parts]
    means = [ops.pool_mean(s[0], 64) for s in shards]
    G = H // Hkv
    for r, (p, (Qs, Ks, Vs, gs)) in enumerate(zip(parts, shards)):
        if p.split == 1:
            out = P.nsa_forward_head_parallel(Qs, Ks, Vs, cfg, gate_logits=gs, group=None)
            want = ref.reshape(B * Hkv, G, T, D)[p.u0:p.u1].reshape(1, -1, T, D)
        else:
            # what the all-gather over the ranks sharing the KV head returns: their block means in head order
            monkeypatch.setattr(P, "gather_heads", lambda x, group, _p=p: torch.cat([means[q] for q in _p.peers], dim=1))
            idx = P.resolve_block_indices_split(Qs, Ks, cfg, "peers", scale=D ** -0.5)
            if shared:
                assert torch.equal(idx, ref_idx[:, p.u0:p.u0 + 1])
            else:
                assert torch.equal(idx, ref_idx.reshape(B * Hkv, G, *ref_idx.shape[2:])[p.u0, p.h0:p.h1].unsqueeze(0))
            out = P.nsa_forward_head_parallel(Qs, Ks, Vs, cfg, gate_logits=gs, group="peers")
            want = ref.reshape(B * Hkv, G, T, D)[p.u0, p.h0:p.h1].unsqueeze(0)
        if (p.h1 - p.h0) % 4 == 0:
            assert torch.equal(out, want), (world, r, float((out.float() - want.float()).abs().max()))
        else:
            # fewer than four heads per rank: the kernel's work item then groups rows differently (two heads x two
            # query blocks instead of four heads x one), and its lazy rescaling decides per warp -- same arithmetic,
            # another reference maximum for some rows, so the 16-bit roundings of P differ in the last place
            assert float((out.float() - want.float()).abs().max()) <= 1e-2
    ops.device_status()
