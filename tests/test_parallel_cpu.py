"""Host-side logic of the multi-GPU layouts on CPU: two gloo ranks.  The oracle stands in for the
kernels (forward_fn), so what is checked is the sharding, the all-gather and the offset geometry."""
import os
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class Cfg:
    block_size_c, stride_c, block_size_n, block_size_m, top_k, window_size = 32, 16, 64, 64, 3, 96
    causal, pool, gate_activation, scale, force_first, force_local, select_per_group = True, "mean", "sigmoid", None, 1, 2, True


def _oracle_forward(Q, K, V, cfg, gate_logits=None):
    from oracle import nsa_oracle as O
    return O.nsa_forward(Q, K, V, block_size_c=cfg.block_size_c, stride_c=cfg.stride_c, top_k=cfg.top_k,
                         window_size=cfg.window_size, gate_logits=gate_logits, force_first=cfg.force_first,
                         force_local=cfg.force_local, group_shared=cfg.select_per_group)


def _inputs():
    g = torch.Generator().manual_seed(3)
    B, H, Hkv, T, D = 1, 4, 2, 256, 32
    Q = torch.randn(B, H, T, D, generator=g).to(torch.bfloat16)
    K = torch.randn(B, Hkv, T, D, generator=g).to(torch.bfloat16)
    V = torch.randn(B, Hkv, T, D, generator=g).to(torch.bfloat16)
    gates = torch.randn(B, H, T, 3, generator=g)
    return Q, K, V, gates


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from nsa_from_scratch_b200 import parallel as P
    Q, K, V, gates = _inputs()
    T = Q.shape[2]
    Tl = T // world
    sl = slice(rank * Tl, (rank + 1) * Tl)
    out = P.nsa_forward_context_parallel(Q[:, :, sl], K[:, :, sl], V[:, :, sl], Cfg, gate_logits=gates[:, :, sl],
                                         forward_fn=_oracle_forward)
    torch.save(out, os.path.join(out_dir, f"cp_{rank}.pt"))
    Qs, Ks, Vs, gs = P.shard_kv_heads(Q, K, V, world, rank, gates)
    torch.save(_oracle_forward(Qs, Ks, Vs, Cfg, gate_logits=gs), os.path.join(out_dir, f"hp_{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_context_and_head_parallel_layouts_match_single_rank(tmp_path):
    world, port = 2, 29517 + os.getpid() % 200
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    Q, K, V, gates = _inputs()
    ref = _oracle_forward(Q, K, V, Cfg, gate_logits=gates)
    cp = torch.cat([torch.load(tmp_path / f"cp_{r}.pt") for r in range(world)], dim=2)
    assert torch.allclose(cp, ref, atol=1e-5), float((cp - ref).abs().max())
    hp = torch.cat([torch.load(tmp_path / f"hp_{r}.pt") for r in range(world)], dim=1)
    assert torch.allclose(hp, ref, atol=1e-5), float((hp - ref).abs().max())


def test_unit_range_is_a_balanced_partition():
    from nsa_from_scratch_b200.parallel import unit_range
    for n in (1, 4, 7, 64):
        for w in (1, 2, 3, 8):
            spans = [unit_range(n, w, r) for r in range(w)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
