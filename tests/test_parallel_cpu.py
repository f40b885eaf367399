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
    # more ranks than KV heads: the query heads of ONE KV head split over the two ranks; the block means they
    # all-gather come back in head order, identical on both ranks
    part = P.head_partition(1, 4, 1, world, rank)
    assert part.split == 2 and part.peers == (0, 1) and (part.h0, part.h1) == (2 * rank, 2 * rank + 2)
    grp = P.head_groups(1, 4, 1, world, rank)
    Q1, K1, V1, g1 = P.shard_heads(Q, K[:, :1], V[:, :1], part, gates)
    assert Q1.shape == (1, 2, T, Q.shape[3]) and torch.equal(Q1[0], Q[0, 2 * rank:2 * rank + 2]) and K1.shape[1] == 1
    means = Q1.float().reshape(1, 2, T // 64, 64, -1).mean(3).to(torch.bfloat16)
    torch.save(P.gather_heads(means, grp), os.path.join(out_dir, f"means_{rank}.pt"))
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


    Qm = Q.float().reshape(1, 4, Q.shape[2] // 64, 64, -1).mean(3).to(torch.bfloat16)
    for r in range(world):
        assert torch.equal(torch.load(tmp_path / f"means_{r}.pt"), Qm)


def _late_worker(rank, world, port, out_dir):
    import time
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from nsa_from_scratch_b200 import parallel as P
    x = torch.full((1, 1, 8, 4), float(rank))
    dist.barrier()
    result = "completed"
    if rank == 1:
        time.sleep(6.0)                          # the late rank: joins long after its peer's limit has passed
    try:
        P.gather_key_prefix(x, timeout_s=1.5)
    except P.ContextParallelTimeout:
        result = "timeout"
    except Exception as e:                       # the peer has gone by the time the late rank arrives
        result = "error:" + type(e).__name__
    open(os.path.join(out_dir, f"late_{rank}.txt"), "w").write(result)
    os._exit(0)                                  # the group is unusable after the failed collective: leave without it


def test_context_parallel_collective_gives_up_on_a_late_rank(tmp_path):
    """A rank that does not join the all-gather within the limit makes the wrapper raise ContextParallelTimeout on
    the waiting rank instead of blocking it forever (failure made on the host: a rank that sleeps)."""
    world, port = 2, 29717 + os.getpid() % 200
    mp.spawn(_late_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    assert (tmp_path / "late_0.txt").read_text() == "timeout"
    assert (tmp_path / "late_1.txt").read_text() != "completed"


def test_head_partition_covers_every_head_once():
    from nsa_from_scratch_b200.parallel import head_partition
    for B, H, Hkv in ((1, 64, 4), (2, 12, 1), (1, 16, 16), (2, 8, 2)):
        G = H // Hkv
        for world in (1, 2, 4, 8, 16):
            try:
                parts = [head_partition(B, H, Hkv, world, r) for r in range(world)]
            except ValueError:
                assert world > B * Hkv and (world % (B * Hkv) or G % (world // (B * Hkv)))
                continue
            seen = set()
            for p in parts:
                for u in range(p.u0, p.u1):
                    for h in range(p.h0, p.h1):
                        assert (u, h) not in seen
                        seen.add((u, h))
                assert len(p.peers) == p.split and (p.split == 1 or all(parts[q].u0 == p.u0 for q in p.peers))
            assert len(seen) == B * Hkv * G
    p = head_partition(1, 64, 4, 8, 5)               # the benchmark shape on 8 GPUs: KV head 2, second half of its 16 heads
    assert (p.u0, p.u1, p.h0, p.h1, p.split, p.peers) == (2, 3, 8, 16, 2, (4, 5))


def test_unit_range_is_a_balanced_partition():
    from nsa_from_scratch_b200.parallel import unit_range
    for n in (1, 4, 7, 64):
        for w in (1, 2, 3, 8):
            spans = [unit_range(n, w, r) for r in range(w)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
