"""Decoding against a growing KV cache: parity with the oracle's Tq < Tk forward (the reference's own
tail-aligned convention) and with the full-sequence forward on block-aligned chunks."""
import pytest
import torch

from helpers import make_qkv, max_abs
from oracle import nsa_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def nsa():
    import nsa_from_scratch_b200 as m
    return m


CFGS = {
    "stride16": dict(block_size_c=32, stride_c=16, top_k=3, window_size=96, force_first=1, force_local=1, select_per_group=True),
    "reference_geometry": dict(block_size_c=64, top_k=2, window_size=64),
}


@pytest.mark.parametrize("cfg_name", list(CFGS))
@pytest.mark.parametrize("D", [64, 128])
def test_decode_steps_vs_oracle(nsa, cfg_name, D):
    """Prefill of 200 positions, then single-token and ragged multi-token steps; every step against the oracle
    called on the filled prefix (Tq < Tk).  The cache is longer than what is filled."""
    kw = CFGS[cfg_name]
    B, H, Hkv, T = 2, 8, 2, 333
    Q, K, V, g = make_qkv(41, B, H, Hkv, T, T, D)
    gates = torch.randn(B, H, T, 3, generator=g)
    cfg = nsa.NSAConfig(**kw)
    cache = nsa.KVCache(B, Hkv, D, 512, cfg)
    Qc, Kc, Vc, Gc = Q.cuda(), K.cuda(), V.cuda(), gates.cuda()
    okw = dict(block_size_c=kw["block_size_c"], stride_c=kw.get("stride_c"), top_k=kw["top_k"], window_size=kw["window_size"],
               force_first=kw.get("force_first", 0), force_local=kw.get("force_local", 0), group_shared=kw.get("select_per_group", False))
    pos = 0
    for step in (200, 1, 1, 1, 61, 1, 7, 64, 1):
        if pos + step > T:
            break
        cache.append(Kc[:, :, pos:pos + step], Vc[:, :, pos:pos + step])
        pos += step
        assert cache.length == pos
        out = nsa.nsa_decode(Qc[:, :, pos - step:pos], cache, gate_logits=Gc[:, :, pos - step:pos], nsplit=1)
        # the pooled tensors and block means the cache keeps are those a fresh computation gives
        from nsa_from_scratch_b200 import ops
        n = cache.n_pooled(pos)
        if n:
            assert torch.equal(cache.Kc[:, :, :n], ops.pool_mean(Kc[:, :, :pos], cache.bc, cache.stride))
        assert torch.equal(cache.Kb[:, :, :(pos + 63) // 64], ops.pool_mean(Kc[:, :, :pos], 64, 64))
        idx = O.select_blocks(Q[:, :, pos - step:pos].float(), K[:, :, :pos].float(), top_k=kw["top_k"],
                              force_first=okw["force_first"], force_local=okw["force_local"], group_shared=okw["group_shared"])
        ref = O.nsa_forward(Q[:, :, pos - step:pos].float(), K[:, :, :pos].float(), V[:, :, :pos].float(),
                            gate_logits=gates[:, :, pos - step:pos], block_indices=idx, **okw)
        assert max_abs(out, ref) <= 2e-2, (step, pos, max_abs(out, ref))
        # and what the ordinary forward returns for the same call
        full = nsa.nsa_forward(Qc[:, :, pos - step:pos], Kc[:, :, :pos].contiguous(), Vc[:, :, :pos].contiguous(), cfg,
                               gate_logits=Gc[:, :, pos - step:pos].contiguous())
        assert torch.equal(out, full)


@pytest.mark.parametrize("D,dtype", [(128, torch.bfloat16), (64, torch.float16)])
@pytest.mark.parametrize("nsplit", [2, 5, 16, None])
def test_split_launch_vs_oracle_and_unsplit(nsa, D, dtype, nsplit):
    """Key tiles of a work item spread over several thread blocks and merged: against the oracle and
    against the ordinary launch (not bit-equal: the partial sums are merged in fp32 and rounded once)."""
    B, H, Hkv, Tk = 1, 8, 2, 2100
    cfg = nsa.NSAConfig(block_size_c=32, stride_c=16, top_k=4, window_size=200, force_first=1, force_local=2, select_per_group=True)
    Q, K, V, g = make_qkv(47, B, H, Hkv, Tk, Tk, D, dtype=dtype)
    gates = torch.randn(B, H, Tk, 3, generator=g)
    cache = nsa.KVCache(B, Hkv, D, 2304, cfg, dtype=dtype)
    cache.append(K.cuda(), V.cuda())
    for Tq in (1, 3, 70):
        q, gl = Q[:, :, Tk - Tq:].cuda(), gates[:, :, Tk - Tq:].cuda()
        one = nsa.nsa_decode(q, cache, gate_logits=gl, nsplit=1)
        out = nsa.nsa_decode(q, cache, gate_logits=gl, nsplit=nsplit)
        assert max_abs(out, one) <= 1e-2, (Tq, max_abs(out, one))
        idx = O.select_blocks(Q[:, :, Tk - Tq:].float(), K.float(), top_k=4, force_first=1, force_local=2, group_shared=True)
        ref = O.nsa_forward(Q[:, :, Tk - Tq:].float(), K.float(), V.float(), gate_logits=gates[:, :, Tk - Tq:], block_indices=idx,
                            block_size_c=32, stride_c=16, top_k=4, window_size=200, force_first=1, force_local=2, group_shared=True)
        assert max_abs(out, ref) <= 2e-2, (Tq, max_abs(out, ref))
    from nsa_from_scratch_b200 import ops
    ops.device_status()


@pytest.mark.parametrize("cfg_name", list(CFGS))
def test_graphed_decoder_equals_eager_steps(nsa, cfg_name):
    """The decoding step as one CUDA graph with the fill count in device memory: 70 replays (crossing
    compression-window and selection-block boundaries) against eager steps on a second cache."""
    kw = CFGS[cfg_name]
    B, H, Hkv, D, T0, steps = 2, 8, 2, 128, 150, 70
    Q, K, V, g = make_qkv(53, B, H, Hkv, T0 + steps, T0 + steps, D)
    gates = torch.randn(B, H, T0 + steps, 3, generator=g)
    cfg = nsa.NSAConfig(**kw)
    Qc, Kc, Vc, Gc = Q.cuda(), K.cuda(), V.cuda(), gates.cuda()
    ca, cb = nsa.KVCache(B, Hkv, D, 256, cfg), nsa.KVCache(B, Hkv, D, 256, cfg)
    ca.append(Kc[:, :, :T0], Vc[:, :, :T0])
    cb.append(Kc[:, :, :T0], Vc[:, :, :T0])
    dec = nsa.GraphedDecoder(ca, H, nsplit=3)
    assert ca.length == T0 and int(ca.filled_dev.item()) == T0
    for t in range(T0, T0 + steps):
        dec.q.copy_(Qc[:, :, t:t + 1]); dec.k.copy_(Kc[:, :, t:t + 1]); dec.v.copy_(Vc[:, :, t:t + 1])
        dec.gate_logits.copy_(Gc[:, :, t:t + 1])
        out = dec.step()
        cb.append(Kc[:, :, t:t + 1], Vc[:, :, t:t + 1])
        ref = nsa.nsa_decode(Qc[:, :, t:t + 1], cb, gate_logits=Gc[:, :, t:t + 1], nsplit=3)
        assert torch.equal(out, ref), (t, max_abs(out, ref))
    assert ca.length == T0 + steps == int(ca.filled_dev.item())
    n = ca.n_pooled(ca.length)
    assert torch.equal(ca.Kc[:, :, :n], cb.Kc[:, :, :n]) and torch.equal(ca.Kb, cb.Kb) and torch.equal(ca.K, cb.K)
    # eager use of the same cache keeps the device count current
    ca.reset()
    assert int(ca.filled_dev.item()) == 0
    with pytest.raises(ValueError):
        ca.length = 256
        dec.step()
    from nsa_from_scratch_b200 import ops
    ops.device_status()


def test_chunked_prefill_equals_full_forward(nsa):
    """Block-aligned chunks through the cache reproduce the rows of one full-sequence forward."""
    B, H, Hkv, T, D = 1, 8, 2, 512, 128
    Q, K, V, g = make_qkv(43, B, H, Hkv, T, T, D)
    cfg = nsa.NSAConfig(block_size_c=32, stride_c=16, top_k=3, window_size=96, force_first=1, force_local=1, select_per_group=True)
    Qc, Kc, Vc = Q.cuda(), K.cuda(), V.cuda()
    full = nsa.nsa_forward(Qc, Kc, Vc, cfg)
    cache = nsa.KVCache(B, Hkv, D, 1024, cfg)
    for c0 in range(0, T, 128):
        cache.append(Kc[:, :, c0:c0 + 128], Vc[:, :, c0:c0 + 128])
        out = nsa.nsa_decode(Qc[:, :, c0:c0 + 128].contiguous(), cache, nsplit=1)
        assert torch.equal(out, full[:, :, c0:c0 + 128])
    cache.reset()
    assert cache.length == 0
    with pytest.raises(ValueError):
        cache.append(Kc[:, :, :1], Vc[:, :, :1]); cache.append(torch.zeros(B, Hkv, 1024, D, dtype=torch.bfloat16, device="cuda"),
                                                            torch.zeros(B, Hkv, 1024, D, dtype=torch.bfloat16, device="cuda"))
