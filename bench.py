"""NSA forward throughput benchmark.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--seq-len T] ...

One "step" is one NSA forward (pool K/V, pool block means, score + top-k, fused three-branch
attention with the gated combine) over one synthetic batch.  Default workload: bf16, B=1,
T=65536 causal, Hq=64, Hkv=4, D=128, compression block 32 / stride 16, selection block 64 with
top-16 (block 0 and the 2 local blocks forced), window 512, sigmoid gates from a random
Linear(D,3) applied to Q.  With N GPUs (--layout heads, the default) that ONE problem is split by
(batch, KV head) units -- whole KV heads per rank up to 4 GPUs, no collective; on 8 GPUs the 16 query heads of a
KV head are split over two ranks, which all-gather their query block means (2 MB) so that the group-shared
block lists stay bit-exact -- strong scaling, value = T / max-rank time.  With N > 1 the line also carries a
`context_parallel` block: T=262144 sharded contiguously by query position, K/V all-gathered over NCCL.
--layout replicas gives every rank its own batch element instead (weak scaling, no collective).

Prints ONE JSON line (rank 0).  `--impl reference` times the CPU oracle port (the reference's
plain-torch algorithm) on a bounded sample of the same workload on the host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

METRIC = "nsa_fwd_tokens_per_s"
UNIT = "tokens/s"


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--seq-len", type=int, default=65536)
    ap.add_argument("--heads", type=int, default=64)
    ap.add_argument("--kv-heads", type=int, default=4)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--cmp-block", type=int, default=32)
    ap.add_argument("--cmp-stride", type=int, default=16)
    ap.add_argument("--top-k", type=int, default=16)
    ap.add_argument("--window", type=int, default=512)
    ap.add_argument("--engine", default="auto", choices=["auto", "generic", "tcgen05"])
    ap.add_argument("--select", default="group", choices=["group", "head"],
                    help="block lists shared by the query heads of a KV head (group) or one per query head (head)")
    ap.add_argument("--layout", default="heads", choices=["heads", "replicas", "cp"],
                    help="heads: ONE B=1 problem split over the ranks by (batch, KV head) units and, beyond that, by query "
                         "heads inside a group (strong scaling); replicas: every rank runs the whole workload on its own "
                         "batch element (weak scaling); cp: context parallel, --seq-len is the TOTAL length, queries sharded "
                         "contiguously, K/V all-gathered over NCCL inside the timed step (strong scaling)")
    ap.add_argument("--cp-seq-len", type=int, default=262144,
                    help="total length of the context-parallel measurement appended to the line when N > 1 (0 = leave it out)")
    ap.add_argument("--sweep", action="store_true",
                    help="instead of the single contract line: one JSON line per point of the T x D sweep "
                         "(T = 1k..64k, D = 64/128, Hq=64/Hkv=4) plus the reference's own MHA shape (H=16, D=64, 64/64)")
    ap.add_argument("--train", action="store_true", help="only the training-shape measurements of --sweep (at --seq-len if given below 32768)")
    ap.add_argument("--scorer", action="store_true", help="only the probability-scorer measurement of --sweep")
    ap.add_argument("--decode", action="store_true", help="only the decoding measurement of --sweep (B=1, 65536 cached)")
    ap.add_argument("--cpu-tiles", type=int, default=40, help="64-row query tiles in the CPU-baseline sample")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--host-chunk", type=int, default=16384,
                    help="query positions per pipeline unit of the host-tensor entry point (0 = whole sequences)")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--protocol", default="contract", choices=["contract", "reference"],
                    help="reference: the reference benchmark's own protocol (25 warm-up + 100 timed iterations per seed, "
                         "seeds 0,1,2, one event pair per iteration, pooled mean and a 95 %% percentile-bootstrap interval)")
    return ap.parse_args()


def workload_name(a):
    return (f"nsa_fwd bf16 B=1 T={a.seq_len} Hq={a.heads} Hkv={a.kv_heads} D={a.head_dim} "
            f"cmp={a.cmp_block}/{a.cmp_stride} sel=64x{a.top_k}(forced 1+2, per {a.select}) win={a.window} sigmoid-gates")


def make_inputs(a, seed, heads=None, kv_heads=None, rows=None):
    """Q, K, V ~ N(0,1) bf16 and gate logits = Linear(D,3)(Q) from CPU generators.  Every query head and every KV
    head has a generator of its own (seeded by `seed` and the head's number), so a rank that holds some heads of the
    problem builds exactly the values the whole problem has; the gate weights come from `seed` alone.
    `heads` / `kv_heads`: the global head numbers wanted (default: all); `rows`: (first, last+1) of the sequence."""
    B, T, D = 1, a.seq_len, a.head_dim
    heads = list(range(a.heads)) if heads is None else list(heads)
    kv_heads = list(range(a.kv_heads)) if kv_heads is None else list(kv_heads)
    r0, r1 = (0, T) if rows is None else rows
    bound = 1.0 / D ** 0.5                                           # torch.nn.Linear default init range
    Wg = (torch.rand(3, D, generator=torch.Generator().manual_seed(seed * 1000003 + 7)) * 2 - 1) * bound
    Q = torch.empty(B, len(heads), r1 - r0, D, dtype=torch.bfloat16)
    gates = torch.empty(B, len(heads), r1 - r0, 3, dtype=torch.bfloat16)
    for i, h in enumerate(heads):
        q = torch.randn(T, D, generator=torch.Generator().manual_seed(seed * 1000003 + 1000 + h))[r0:r1].to(torch.bfloat16)
        Q[0, i] = q
        gates[0, i] = (q.float() @ Wg.t()).to(torch.bfloat16)
    K = torch.empty(B, len(kv_heads), r1 - r0, D, dtype=torch.bfloat16)
    V = torch.empty(B, len(kv_heads), r1 - r0, D, dtype=torch.bfloat16)
    for i, h in enumerate(kv_heads):
        g = torch.Generator().manual_seed(seed * 1000003 + 500000 + h)
        K[0, i] = torch.randn(T, D, generator=g)[r0:r1].to(torch.bfloat16)
        V[0, i] = torch.randn(T, D, generator=g)[r0:r1].to(torch.bfloat16)
    return Q, K, V, gates


# ------------------------------------------------------------------ CPU baseline (oracle port)
def cpu_sample(a, n_tiles, repeats=1):
    """Times the CPU oracle on `n_tiles` 64-row query tiles (all heads) spread evenly over the
    sequence; each tile sees its full causal prefix of keys.  Returns (tokens/s, seconds, description)."""
    from oracle import nsa_oracle as O
    torch.set_num_threads(os.cpu_count() or 1)
    Q, K, V, gates = make_inputs(a, a.seed)
    T = a.seq_len
    nq = T // 64
    tiles = sorted({min(nq - 1, int((i + 0.5) * nq / n_tiles)) for i in range(n_tiles)})
    best = None
    for _ in range(repeats):
        t0 = time.perf_counter()
        for qb in tiles:
            q0, q1 = qb * 64, (qb + 1) * 64
            O.nsa_forward(Q[:, :, q0:q1], K[:, :, :q1], V[:, :, :q1], block_size_c=a.cmp_block,
                          stride_c=a.cmp_stride, top_k=a.top_k, window_size=a.window,
                          gate_logits=gates[:, :, q0:q1].float(), force_first=1, force_local=2,
                          group_shared=a.select == "group")
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    toks = len(tiles) * 64
    return toks / best, best, f"{len(tiles)} query tiles of 64 rows x {a.heads} heads at blocks {tiles}, full causal key prefix each"


def run_reference(a):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    n_tiles = max(2, a.cpu_tiles)
    times = []
    for _ in range(a.warmup if a.warmup < 2 else 1):
        cpu_sample(a, 2)
    val = None
    for _ in range(max(1, min(a.steps, 3))):
        v, dt, desc = cpu_sample(a, n_tiles)
        times.append(dt)
        val = v if val is None else max(val, v)
    cores = torch.get_num_threads()
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": a.gpus, "steps": len(times),
        "warmup": 1, "ms_per_step": 1e3 * min(times), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(a), "note": "CPU oracle port of the reference's plain-torch path"},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": cores, "kind": "port", "sample": desc},
        "cpu_baseline_reference_native": native_reference_cpu(a.seed),
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------ clocks
class ClockSampler:
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.rows, self.proc = [], None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "50", "-i", str(index)], stdout=subprocess.PIPE, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append(line.strip().split(", "))

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            pass
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 7:
                continue
            try:
                sm.append(float(r[0]))
                mx = float(r[1])
            except ValueError:
                continue
            for n, v in zip(names, r[3:7]):
                if v.strip().lower() == "active":
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


# ------------------------------------------------------------------ ours
def algorithmic_flops(a, idx):
    """4*D*(unmasked q,k pairs) per branch, summed over heads; selected pairs from the index tensor."""
    T, D, H = a.seq_len, a.head_dim, a.heads
    l, d, W = a.cmp_block, a.cmp_stride, a.window
    t = torch.arange(T, dtype=torch.int64)
    n_c = (T - l) // d + 1 if d != l else -(-T // l)
    vis = torch.clamp((t - (l - 1)) // d + 1, min=0, max=n_c)
    vis = torch.where(t - (l - 1) >= 0, vis, torch.zeros_like(vis))
    cmp_pairs = int(vis.sum()) * H
    sld_pairs = int(torch.clamp(t + 1, max=W).sum()) * H
    nq = idx.shape[2]
    qb = torch.arange(nq, device=idx.device).view(1, 1, nq, 1)
    full = (idx < qb) & (idx >= 0)
    diag = idx == qb
    sel_pairs = int(full.sum()) * 64 * 64 + int(diag.sum()) * (64 * 65 // 2)
    if idx.shape[1] != H:
        sel_pairs *= H // idx.shape[1]
    f = lambda p: 4.0 * D * p
    return {"compressed": f(cmp_pairs), "selected": f(sel_pairs), "sliding": f(sld_pairs),
            "total": f(cmp_pairs + sel_pairs + sld_pairs)}


def measured_peaks():
    try:
        return json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        return {}


def native_reference_cpu(seed):
    """The reference's own plain-torch forward (nsa_attention_reference), unmodified, on its CPU-runnable case:
    fp32, B=1, T=4096, Hq=16 query heads sharing one KV head (expanded to 16: it has no grouped heads), D=64,
    its own geometry (64-token compression blocks, plain top-16, window 512), gates = sigmoid(Linear(D,3)(Q)).
    Needs oracle/_ref (made by oracle/make_ref.py where a checkout exists); returns None without it."""
    path = os.path.join(ROOT, "oracle", "_ref", "nsa_reference.py")
    if not os.path.isfile(path):
        return None
    import importlib.util
    spec = importlib.util.spec_from_file_location("nsa_reference_native", path)
    ref = importlib.util.module_from_spec(spec)
    sys.modules["nsa_reference_native"] = ref      # dataclasses look their module up by name
    spec.loader.exec_module(ref)
    torch.set_num_threads(os.cpu_count() or 1)
    g = torch.Generator().manual_seed(seed)
    T, H, D = 4096, 16, 64
    Q = torch.randn(1, H, T, D, generator=g)
    K = torch.randn(1, 1, T, D, generator=g).expand(1, H, T, D).contiguous()
    V = torch.randn(1, 1, T, D, generator=g).expand(1, H, T, D).contiguous()
    Wg = (torch.rand(3, D, generator=g) * 2 - 1) / D ** 0.5
    gates = torch.einsum("bhtd,cd->bhtc", Q, Wg)
    cfg = ref.NSAConfig()
    ts, out = [], None
    for i in range(4):
        t0 = time.perf_counter()
        out = ref.nsa_attention_reference(Q, K, V, cfg, gates=gates)
        if i > 0:
            ts.append(time.perf_counter() - t0)
    med = statistics.median(ts)
    return {"value": T / med, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "reference",
            "sample": f"nsa_attention_reference, fp32, B=1 T={T} H={H} (one KV head expanded) D={D}, 64/64 compression, top-16, "
                      f"window 512; median of {len(ts)} runs after 1 warm-up",
            "seconds": med, "rows_without_any_key_nan": int((~torch.isfinite(out).all(-1)).sum())}


def run_ours(a):
    import nsa_from_scratch_b200 as nsa
    from nsa_from_scratch_b200 import _lib as L, forward as F, ops, parallel

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU path for --impl ours)"
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if dist is None:
            return ms
        t_ = torch.tensor([ms], device="cuda")
        dist.all_reduce(t_, op=dist.ReduceOp.MAX)
        return float(t_.item())

    cfg = nsa.NSAConfig(block_size_c=a.cmp_block, stride_c=a.cmp_stride, block_size_n=64, block_size_m=64,
                        top_k=a.top_k, window_size=a.window, force_first=1, force_local=2,
                        select_per_group=a.select == "group")
    engine = {"auto": L.ENGINE_AUTO, "generic": L.ENGINE_GENERIC, "tcgen05": L.ENGINE_TCGEN05}[a.engine]
    ops.set_engine(a.engine)
    if a.layout == "cp":
        line = run_cp(a, a.seq_len, nsa, cfg, rank, world, dist, barrier, max_over_ranks, a.steps, a.warmup)
        if rank == 0:
            print(json.dumps(line), flush=True)
        if dist is not None:
            dist.destroy_process_group()
        return
    T, D, H, Hkv = a.seq_len, a.head_dim, a.heads, a.kv_heads
    scale = D ** -0.5
    shared = a.select == "group"
    group = None
    if a.layout == "heads":
        # ONE problem: this rank's (batch, KV head) units, or its share of the query heads of one unit
        part = parallel.head_partition(1, H, Hkv, world, rank)
        if world > 1:
            group = parallel.head_groups(1, H, Hkv, world, rank)
        G_ = H // Hkv
        q_heads = [u * G_ + h for u in range(part.u0, part.u1) for h in range(part.h0, part.h1)]
        kv_list = list(range(part.u0, part.u1))
        Qh, Kh, Vh, Gh = make_inputs(a, a.seed, heads=q_heads, kv_heads=kv_list)
        tokens_total, scaling = T, "strong"
        par = (f"one B=1 problem over {world} rank(s): {len(kv_list)} KV head(s) x {part.h1 - part.h0} query heads per rank"
               + (f", query block means all-gathered among the {part.split} ranks of a KV head" if part.split > 1 and shared else ", no collective"))
    else:
        Qh, Kh, Vh, Gh = make_inputs(a, a.seed + rank)
        tokens_total, scaling = world * T, "weak"
        par = f"replicas: every rank its own batch element, {world} rank(s), no collective"
    Qh, Kh, Vh, Gh = (t.pin_memory() for t in (Qh, Kh, Vh, Gh))
    Q, K, V, G = (t.cuda(non_blocking=True) for t in (Qh, Kh, Vh, Gh))
    torch.cuda.synchronize()

    def step():
        # the public entry point (selection inside); a rank that shares its KV head goes through the layout's wrapper
        if group is not None:
            return parallel.nsa_forward_head_parallel(Q, K, V, cfg, gate_logits=G, group=group)
        return nsa.nsa_forward(Q, K, V, cfg, gate_logits=G)
    LAUNCHES_PER_STEP = 6   # pool Q means, pool K means, select, pool K, pool V, fused attention

    for _ in range(a.warmup):
        out = step()
    barrier()

    # ---- timed region: K steps, CUDA events, max over ranks -----------------------------
    sampler = ClockSampler(local) if rank == 0 else None
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    barrier()
    ev[0].record()
    for _ in range(a.steps):
        out = step()
    ev[1].record()
    barrier()
    ms_step = max_over_ranks(ev[0].elapsed_time(ev[1])) / a.steps
    value = tokens_total / (ms_step * 1e-3)

    # ---- per-kernel timing of the dominant (fused attention) kernel on this rank's share ------------------
    def indices():
        if group is not None:
            return parallel.resolve_block_indices_split(Q, K, cfg, group, scale=scale)
        return F._resolve_block_indices(Q, K, block_size_m=64, block_size_n=64, top_k=a.top_k, causal=True, scale=scale,
                                        force_first=1, force_local=2, shared_per_group=shared)
    import copy
    mine = copy.copy(a)
    mine.heads, mine.kv_heads = Q.shape[1], K.shape[1]
    idx = indices()
    flops = algorithmic_flops(mine, idx)
    stage_ms = {"pool_select": [], "fused_attention": []}
    for _ in range(a.steps):
        e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        e[0].record()
        idx = indices()
        Kc = ops.pool_mean(K, a.cmp_block, a.cmp_stride)
        Vc = ops.pool_mean(V, a.cmp_block, a.cmp_stride)
        e[1].record()
        ops.attention_fwd(Q, K, V, branches=7, fused=True, causal=True, scale=scale, Kc=Kc, Vc=Vc,
                          cmp_block=a.cmp_block, cmp_stride=a.cmp_stride,
                          cmp_offset=(Kc.shape[2] * a.cmp_block if a.cmp_stride == a.cmp_block else T) - T,
                          idx=idx, bm=64, bn=64, window=a.window, gates=G, engine=engine)
        e[2].record()
        torch.cuda.synchronize()
        stage_ms["pool_select"].append(e[0].elapsed_time(e[1]))
        stage_ms["fused_attention"].append(e[1].elapsed_time(e[2]))
    # each branch alone through the same kernel (unfused: writes its own output and lse), for a
    # per-branch share of the roofline; a few launches each, not part of the step
    branch_ms = {}
    Kc = ops.pool_mean(K, a.cmp_block, a.cmp_stride)
    Vc = ops.pool_mean(V, a.cmp_block, a.cmp_stride)
    for name, bit in (("compressed", 1), ("selected", 2), ("sliding", 4)):
        ts = []
        for i in range(4):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            ops.attention_fwd(Q, K, V, branches=bit, fused=False, causal=True, scale=scale, Kc=Kc, Vc=Vc,
                              cmp_block=a.cmp_block, cmp_stride=a.cmp_stride,
                              cmp_offset=(Kc.shape[2] * a.cmp_block if a.cmp_stride == a.cmp_block else T) - T,
                              idx=idx, bm=64, bn=64, window=a.window, engine=engine)
            e1.record()
            torch.cuda.synchronize()
            if i > 0:
                ts.append(e0.elapsed_time(e1))
        branch_ms[name] = statistics.mean(ts)
    # the clock sampler ran through the timed region and the per-kernel timing loops (same kernels, same load)
    clocks = sampler.stop() if sampler else None
    fused_ms = statistics.mean(stage_ms["fused_attention"])
    peaks = measured_peaks()
    # the kernel is timed launch by launch (an event pair and a synchronize around each), the conditions of the burst
    # figure; the sustained figure (seconds of back-to-back GEMMs under the power cap) is kept as a second key
    peak = peaks.get("bf16_tflops")
    peak_src = "measured (burst cuBLAS bf16, MEASURED_PEAKS.json)"
    if peak is None:
        peak, peak_src = 1590.0, "fallback"
    achieved = flops["total"] / (fused_ms * 1e-3) / 1e12
    # DRAM bytes per launch of the fused kernel: dram__bytes_read + dram__bytes_write of one ncu capture at
    # T=16384 with 64 query / 4 KV heads of 128 (572.8 MB), scaled by T and by this rank's share of the heads -- every
    # operand of this shape family grows with both
    traffic = 572.806144e6 * T / 16384 * Q.shape[1] / 64 if (a.heads, a.kv_heads, a.head_dim) == (64, 4, 128) else None
    roofline = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                "traffic": traffic, "traffic_source": "ncu capture at T=16384, scaled (profiles/)", "peak_source": peak_src,
                "kernel": "fused three-branch attention (nsa_fwd_tc5_kernel)" + (f", rank 0's {Q.shape[1]} of {H} heads" if world > 1 and a.layout == "heads" else ""),
                "kernel_ms": fused_ms, "algorithmic_tflop": {k: v / 1e12 for k, v in flops.items()},
                "frac_of_sustained_peak": achieved / peaks["bf16_tflops_sustained"] if "bf16_tflops_sustained" in peaks else None,
                "pool_select_ms": statistics.mean(stage_ms["pool_select"]),
                "branches_alone": {k: {"ms": branch_ms[k], "tflops": flops[k] / (branch_ms[k] * 1e-3) / 1e12,
                                       "frac": flops[k] / (branch_ms[k] * 1e-3) / 1e12 / peak} for k in branch_ms}}

    # ---- end to end: pinned host buffers in, host buffer out, copies inside the timed region ------
    e2e = None
    if not a.no_e2e:
        out_h = torch.empty(out.shape, dtype=out.dtype).pin_memory()
        idx_fn = (lambda qd, kd: parallel.resolve_block_indices_split(qd, kd, cfg, group, scale=scale)) if group is not None else None

        def e2e_step():
            # the public host-tensor entry point: copies in, kernels and copy out pipelined per
            # (batch, KV head, query chunk); it returns when the result is in host memory
            nsa.nsa_forward_host(Qh, Kh, Vh, cfg, gate_logits=Gh, out=out_h, chunk_rows=a.host_chunk or None,
                                 block_indices_fn=idx_fn)
        for _ in range(2):
            e2e_step()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n_e2e = max(2, min(a.steps, 5))
        e0.record()
        for _ in range(n_e2e):
            e2e_step()
        e1.record()
        barrier()
        ms = max_over_ranks(e0.elapsed_time(e1))
        h2d = sum(t.numel() * t.element_size() for t in (Qh, Kh, Vh, Gh))
        e2e = {"value": tokens_total / (ms / n_e2e * 1e-3), "unit": UNIT, "h2d_bytes_per_step": h2d,
               "d2h_bytes_per_step": out_h.numel() * out_h.element_size(), "ms_per_step": ms / n_e2e,
               "bytes_are": "per rank" if world > 1 else "whole job"}
        del out_h

    cpu = cpu_native = None
    if rank == 0 and world == 1 and not a.no_cpu_baseline:
        v, dt, desc = cpu_sample(a, a.cpu_tiles)
        cpu = {"value": v, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port", "sample": desc,
               "seconds": dt}
        cpu_native = native_reference_cpu(a.seed)
    ops.device_status()

    # ---- context parallel at its own length, same process group (N > 1) ---------------------------------
    cp_block = None
    if world > 1 and a.layout == "heads" and a.cp_seq_len > 0 and a.cp_seq_len % (world * 64) == 0:
        del Q, K, V, G, Qh, Kh, Vh, Gh, out, Kc, Vc, idx
        torch.cuda.empty_cache()
        cp_line = run_cp(a, a.cp_seq_len, nsa, cfg, rank, world, dist, barrier, max_over_ranks, max(2, min(a.steps, 3)), 1)
        cp_block = {k: cp_line[k] for k in ("value", "unit", "ms_per_step", "seq_len", "per_rank_ms", "per_rank_forward_alone_ms", "all_gather_ms",
                                              "bytes_received_per_rank", "imbalance_last_over_mean", "steps")} if rank == 0 else None

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": a.steps, "warmup": a.warmup,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": scaling, "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": {"workload": workload_name(a), "global_batch": 1 if a.layout == "heads" else world, "seq_len": T,
                       "parallelism": par, "layout": a.layout,
                       "l2": "inputs (Q alone 1 GiB at the default size) exceed the 126 MB L2", "engine": a.engine},
            "roofline": roofline, "cpu_baseline": cpu, "cpu_baseline_reference_native": cpu_native, "e2e": e2e,
            "clocks": clocks, "gpu_launches": LAUNCHES_PER_STEP * a.steps, "context_parallel": cp_block,
        }
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def run_cp(a, T, nsa, cfg, rank, world, dist, barrier, max_over_ranks, steps, warmup):
    """Context-parallel layout: rank r holds rows [r*Tl, (r+1)*Tl) of Q / gates / out and of K, V -- slices of ONE
    seeded sequence of length T.  Returns the JSON line (meaningful on rank 0)."""
    import copy
    from nsa_from_scratch_b200 import ops, parallel
    assert T % (world * 64) == 0, "the sequence length must be a multiple of 64 * ranks for the cp layout"
    tot = copy.copy(a)
    tot.seq_len = T
    Tl = T // world
    Q, K, V, G = (t.cuda() for t in make_inputs(tot, a.seed, rows=(rank * Tl, (rank + 1) * Tl)))
    stats = {}

    def step():
        if world > 1:
            return parallel.nsa_forward_context_parallel(Q, K, V, cfg, gate_logits=G, stats=stats)
        return nsa.nsa_forward(Q, K, V, cfg, gate_logits=G)
    for _ in range(warmup):
        out = step()
    barrier()
    sampler = ClockSampler(int(os.environ.get("LOCAL_RANK", "0"))) if rank == 0 else None
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    barrier()
    ev[0].record()
    for _ in range(steps):
        out = step()
    ev[1].record()
    barrier()
    ms_mine = ev[0].elapsed_time(ev[1]) / steps
    clocks = sampler.stop() if sampler else None
    ms_step = max_over_ranks(ms_mine * steps) / steps
    # the collective alone (events around it, every rank in step), and each rank's own time
    ag_ms, per_rank, own = None, [ms_mine], [ms_mine]
    if dist is not None:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for _ in range(steps):
            kp = parallel.gather_key_prefix(K)
            vp = parallel.gather_key_prefix(V)
        e1.record()
        barrier()
        ag_ms = max_over_ranks(e0.elapsed_time(e1)) / steps
        # each rank's forward on its gathered prefix with no collective in the loop: inside the step the ranks are
        # coupled by the all-gather (an early rank waits there for the last one), so the step time hides the imbalance
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n_own = max(1, min(steps, 3))
        nsa.nsa_forward(Q, kp, vp, cfg, gate_logits=G)
        f0.record()
        for _ in range(n_own):
            nsa.nsa_forward(Q, kp, vp, cfg, gate_logits=G)
        f1.record()
        torch.cuda.synchronize()
        del kp, vp
        allms = torch.zeros(2, world, device="cuda")
        allms[0, rank] = ms_mine
        allms[1, rank] = f0.elapsed_time(f1) / n_own
        dist.all_reduce(allms)
        per_rank = [float(x) for x in allms[0].tolist()]
        own = [float(x) for x in allms[1].tolist()]
    ops.device_status()
    kv_bytes = 2 * K.numel() * K.element_size() * (world - 1)
    line = {
        "metric": METRIC, "value": T / (ms_step * 1e-3), "unit": UNIT, "n_gpus": world, "steps": steps,
        "warmup": warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "seq_len": T,
        "per_rank_ms": per_rank, "per_rank_forward_alone_ms": own, "all_gather_ms": ag_ms,
        "bytes_received_per_rank": kv_bytes, "imbalance_last_over_mean": own[-1] / (sum(own) / len(own)),
        "config": {"workload": workload_name(tot) + " [context parallel: total T, contiguous query shards]",
                   "global_batch": 1, "seq_len": T, "parallelism": f"cp{world}: all-gather of K/V ({kv_bytes} B received per rank per step) + local forward",
                   "l2": "inputs exceed the 126 MB L2"},
        "roofline": None, "cpu_baseline": None, "e2e": None, "clocks": clocks,
        "gpu_launches": 6 * steps,
    }
    del Q, K, V, G, out
    torch.cuda.empty_cache()
    return line


def run_sweep(a):
    """One line per sweep point: tokens/s with inputs resident, fused-kernel time and TFLOP/s."""
    import copy
    import nsa_from_scratch_b200 as nsa
    from nsa_from_scratch_b200 import forward as F, ops
    torch.cuda.set_device(0)
    points = [dict(seq_len=T, head_dim=D, heads=64, kv_heads=4, cmp_block=32, cmp_stride=16, select="group")
              for D in (128, 64) for T in (1024, 2048, 4096, 8192, 16384, 32768, 65536)]
    points += [dict(seq_len=T, head_dim=64, heads=16, kv_heads=16, cmp_block=64, cmp_stride=64, select="head")
               for T in (4096, 16384, 65536)]
    for pt in points:
        b = copy.copy(a)
        for k, v in pt.items():
            setattr(b, k, v)
        forced = (1, 2) if b.select == "group" else (0, 0)        # the MHA points use the reference's plain top-k
        cfg = nsa.NSAConfig(block_size_c=b.cmp_block, stride_c=b.cmp_stride, top_k=b.top_k, window_size=b.window,
                            force_first=forced[0], force_local=forced[1], select_per_group=b.select == "group")
        Q, K, V, G = (t.cuda() for t in make_inputs(b, a.seed))
        scale = b.head_dim ** -0.5
        for _ in range(a.warmup):
            nsa.nsa_forward(Q, K, V, cfg, gate_logits=G)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.steps):
            nsa.nsa_forward(Q, K, V, cfg, gate_logits=G)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / a.steps
        idx = F._resolve_block_indices(Q, K, block_size_m=64, block_size_n=64, top_k=b.top_k, causal=True, scale=scale,
                                       force_first=forced[0], force_local=forced[1], shared_per_group=b.select == "group")
        flops = algorithmic_flops(b, idx)["total"]
        ops.device_status()
        ms_graph = None
        if b.seq_len <= 8192:                              # launch-bound sizes: the step replayed as one CUDA graph
            graphed = nsa.GraphedForward(Q, K, V, cfg, gate_logits=G)
            graphed()
            torch.cuda.synchronize()
            e0.record()
            for _ in range(a.steps):
                graphed()
            e1.record()
            torch.cuda.synchronize()
            ms_graph = e0.elapsed_time(e1) / a.steps
            del graphed
        print(json.dumps({"metric": METRIC, "value": b.seq_len / (ms * 1e-3), "unit": UNIT, "ms_per_step": ms,
                          "ms_per_step_cuda_graph": ms_graph,
                          "algorithmic_tflop": flops / 1e12, "tflops_whole_step": flops / (ms * 1e-3) / 1e12,
                          "config": {"workload": workload_name(b)}}), flush=True)
        del Q, K, V, G
        torch.cuda.empty_cache()

    def timed(fn, n):
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n

    sweep_train(a)

    # fp8 storage forward (e4m3, per-tensor absmax scales, 0.1 % outliers x20) at T=32768
    b = copy.copy(a)
    b.seq_len = 32768
    Qh, Kh, Vh, Gh = make_inputs(b, a.seed)
    gq = torch.Generator().manual_seed(a.seed + 1)
    xs = []
    for t in (Qh, Kh, Vh):
        t = t.float()
        t = torch.where(torch.rand(t.shape, generator=gq) < 1e-3, t * 20, t)
        xs.append(t.to(torch.bfloat16).cuda())
    q8, k8, v8 = (nsa.quantize_to_fp8(t) for t in xs)
    cfg = nsa.NSAConfig(block_size_c=b.cmp_block, stride_c=b.cmp_stride, top_k=b.top_k, window_size=b.window,
                        force_first=1, force_local=2, select_per_group=True)
    Gc = Gh.cuda()
    o8 = nsa.nsa_forward_fp8(q8[0], k8[0], v8[0], q8[1], k8[1], v8[1], cfg, gate_logits=Gc)
    deq = [(t.to(torch.bfloat16) * sc) for t, sc in (q8, k8, v8)]
    ob = nsa.nsa_forward(deq[0], deq[1], deq[2], cfg, gate_logits=Gc)
    ms8 = timed(lambda: nsa.nsa_forward_fp8(q8[0], k8[0], v8[0], q8[1], k8[1], v8[1], cfg, gate_logits=Gc), max(2, a.steps // 2))
    msb = timed(lambda: nsa.nsa_forward(deq[0], deq[1], deq[2], cfg, gate_logits=Gc), a.steps)
    ops.device_status()
    print(json.dumps({"metric": "nsa_fwd_fp8_tokens_per_s", "value": b.seq_len / (ms8 * 1e-3), "ms_per_step": ms8,
                      "bf16_same_values_ms": msb, "max_abs_vs_bf16_path": float((o8.float() - ob.float()).abs().max()),
                      "config": {"workload": workload_name(b) + " [fp8 e4m3 storage, dequantised in-kernel]"}}), flush=True)
    del q8, k8, v8, deq, xs, o8, ob, Gc
    torch.cuda.empty_cache()

    # the caller path at the default workload: projection outputs [B,T,H,D] in, [B,T,H*D] out.  "steps of the
    # reference module" = transposes, rotary embedding (fp32), casts, gate permute, nsa_forward, transpose back.
    b = copy.copy(a)
    T, H, Hkv, D = b.seq_len, b.heads, b.kv_heads, b.head_dim
    g = torch.Generator().manual_seed(a.seed)
    q = torch.randn(1, T, H, D, generator=g).to(torch.bfloat16).cuda()
    k = torch.randn(1, T, Hkv, D, generator=g).to(torch.bfloat16).cuda()
    v = torch.randn(1, T, Hkv, D, generator=g).to(torch.bfloat16).cuda()
    gl = torch.randn(1, T, H, 3, generator=g).to(torch.bfloat16).cuda()
    cos, sin = nsa.rope_cache(T, D, 10000.0, "cuda")

    def module_steps():
        qq, kk, vv = (t.transpose(1, 2) for t in (q, k, v))
        c, s_ = cos[None, None], sin[None, None]
        rot = lambda t: torch.cat((-t[..., D // 2:], t[..., :D // 2]), dim=-1)
        qq, kk = qq * c + rot(qq) * s_, kk * c + rot(kk) * s_
        o = nsa.nsa_forward(qq.to(torch.bfloat16), kk.to(torch.bfloat16), vv.to(torch.bfloat16), cfg,
                            gate_logits=gl.permute(0, 2, 1, 3).contiguous())
        return o.transpose(1, 2).contiguous().view(1, T, H * D)
    ms_mod = timed(module_steps, max(2, a.steps // 2))
    ms_tm = timed(lambda: nsa.nsa_attention_token_major(q, k, v, cos, sin, cfg, gate_logits=gl), a.steps)
    ms_rope = timed(lambda: ops.rope_to_heads(q, cos, sin), a.steps)
    ops.device_status()
    rope_bytes = 2 * q.numel() * 2                       # read once, write once, 16-bit (tables stay in L2)
    print(json.dumps({"metric": "nsa_layer_tokens_per_s", "value": T / (ms_tm * 1e-3), "ms_per_step": ms_tm,
                      "reference_module_steps_ms": ms_mod, "rope_to_heads_q_ms": ms_rope,
                      "rope_to_heads_q_gbs": rope_bytes / (ms_rope * 1e-3) / 1e9,
                      "config": {"workload": workload_name(b) + " [projection outputs [B,T,H,D] in, [B,T,H*D] out, rotary embedding inside]"}}),
          flush=True)
    del q, k, v, gl
    torch.cuda.empty_cache()

    sweep_scorer(a)
    sweep_decode(a)


def sweep_train(a, T=32768):
    """Selected-branch forward + backward and the whole forward + backward through autograd at the training shape
    (B=2, Hq=12, Hkv=1, D=64); `T` shortens it for a profiler capture."""
    import nsa_from_scratch_b200 as nsa
    from nsa_from_scratch_b200 import forward as F, ops
    torch.cuda.set_device(0)

    def timed(fn, n):
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n
    # selected-branch forward + backward at the training shape (B=2, T=32768, Hq=12, Hkv=1, D=64)
    g = torch.Generator().manual_seed(a.seed)
    B, H, Hkv, D = 2, 12, 1, 64
    Q = torch.randn(B, H, T, D, generator=g).to(torch.bfloat16).cuda()
    K = torch.randn(B, Hkv, T, D, generator=g).to(torch.bfloat16).cuda()
    V = torch.randn(B, Hkv, T, D, generator=g).to(torch.bfloat16).cuda()
    dO = torch.randn(B, H, T, D, generator=g).to(torch.bfloat16).cuda()
    for shared in (False, True):
        idx = F._resolve_block_indices(Q, K, block_size_m=64, block_size_n=64, top_k=16, causal=True, scale=D ** -0.5,
                                       shared_per_group=shared)
        out, lse = nsa.selected_attention(Q, K, V, block_indices=idx)
        nq = T // 64
        qb = torch.arange(nq, device="cuda").view(1, 1, nq, 1)
        pairs = (int(((idx < qb) & (idx >= 0)).sum()) * 4096 + int((idx == qb).sum()) * 2080) * (H // idx.shape[1])
        ms_f = timed(lambda: nsa.selected_attention(Q, K, V, block_indices=idx), a.steps)
        ms_b = timed(lambda: nsa.selected_backward(dO, Q, K, V, out, lse, idx, block_size_m=64, block_size_n=64, causal=True,
                                                   scale=D ** -0.5, Tq=T, Tk=T, return_fp32=True), a.steps)
        ops.device_status()
        print(json.dumps({"metric": "selected_fwd_bwd_ms", "config": {"workload": f"selected branch B={B} T={T} Hq={H} Hkv={Hkv} D={D} bf16, "
                          f"block lists per {'group' if shared else 'head'}"}, "fwd_ms": ms_f, "bwd_ms": ms_b,
                          "fwd_tflops": 4 * D * pairs / (ms_f * 1e-3) / 1e12, "bwd_tflops": 10 * D * pairs / (ms_b * 1e-3) / 1e12,
                          "tokens_per_s_fwd_bwd": B * T / ((ms_f + ms_b) * 1e-3)}), flush=True)
    # whole forward + backward through autograd (all three branch backward kernels + combine) at the same shape
    cfg_t = nsa.NSAConfig(block_size_c=32, stride_c=16, top_k=16, window_size=512, select_per_group=True)
    Qr, Kr, Vr = (t.clone().requires_grad_(True) for t in (Q, K, V))

    def train_step():
        o = nsa.nsa_forward(Qr, Kr, Vr, cfg_t)
        o.backward(dO)
        Qr.grad = Kr.grad = Vr.grad = None
    ms_t = timed(train_step, max(2, a.steps // 2))
    ops.device_status()
    print(json.dumps({"metric": "nsa_fwd_bwd_tokens_per_s", "value": B * T / (ms_t * 1e-3), "ms_per_step": ms_t,
                      "config": {"workload": f"nsa_forward + backward (autograd, every branch on kernels) B={B} T={T} Hq={H} Hkv={Hkv} D={D} bf16"}}),
          flush=True)
    del Q, K, V, dO, Qr, Kr, Vr
    torch.cuda.empty_cache()


def sweep_scorer(a):
    """Selection scored from the compressed branch's probabilities instead of block means: one JSON line with the
    whole forward and the selection alone."""
    import nsa_from_scratch_b200 as nsa
    from nsa_from_scratch_b200 import ops
    torch.cuda.set_device(0)
    Qs, Ks, Vs, Gs = (t.cuda() for t in make_inputs(a, a.seed))
    cfg_p = nsa.NSAConfig(block_size_c=a.cmp_block, stride_c=a.cmp_stride, top_k=a.top_k, window_size=a.window,
                          force_first=1, force_local=2, select_per_group=True, scorer="compressed")

    def timed(fn, n):
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n
    ms_sel = timed(lambda: nsa.select_blocks_compressed(Qs, Ks, cfg_p), max(2, a.steps // 2))
    ms_fwd = timed(lambda: nsa.nsa_forward(Qs, Ks, Vs, cfg_p, gate_logits=Gs), max(2, a.steps // 2))
    ops.device_status()
    print(json.dumps({"metric": METRIC, "value": a.seq_len / (ms_fwd * 1e-3), "unit": UNIT, "ms_per_step": ms_fwd,
                      "selection_ms": ms_sel,
                      "config": {"workload": workload_name(a) + " [selection scored from the compressed branch's probabilities]"}}),
          flush=True)
    del Qs, Ks, Vs, Gs
    torch.cuda.empty_cache()


def sweep_decode(a, shapes=((1, 65536), (8, 65536), (1, 8192))):
    """Decoding against a KV cache: one new token per step (keys appended, pooled K/V and block means brought up
    to date, selection, split attention launch + merge); one JSON line per (batch, cached length)."""
    import nsa_from_scratch_b200 as nsa
    from nsa_from_scratch_b200 import ops
    torch.cuda.set_device(0)
    b = a
    H, Hkv, D = a.heads, a.kv_heads, a.head_dim
    cfg = nsa.NSAConfig(block_size_c=a.cmp_block, stride_c=a.cmp_stride, top_k=a.top_k, window_size=a.window,
                        force_first=1, force_local=2, select_per_group=True)
    for B, Tk in shapes:
        cache = nsa.KVCache(B, Hkv, D, Tk + 256, cfg)
        g = torch.Generator().manual_seed(a.seed)
        for c0 in range(0, Tk - 1, 8192):
            n = min(8192, Tk - 1 - c0)
            cache.append(torch.randn(B, Hkv, n, D, generator=g).to(torch.bfloat16).cuda(),
                         torch.randn(B, Hkv, n, D, generator=g).to(torch.bfloat16).cuda())
        q1 = torch.randn(B, H, 1, D, generator=g).to(torch.bfloat16).cuda()
        k1 = torch.randn(B, Hkv, 1, D, generator=g).to(torch.bfloat16).cuda()
        g1 = torch.randn(B, H, 1, 3, generator=g).cuda()

        def decode_step(ns=None):
            cache.length = Tk - 1                          # the same position every time: the cache does not grow
            cache.append(k1, k1)
            return nsa.nsa_decode(q1, cache, gate_logits=g1, nsplit=ns)
        big = torch.randn(8192, 8192, device="cuda", dtype=torch.bfloat16)

        def device_us(fn, n=20):
            """Device time per call with the host's launch work hidden: a few ms of matmuls go first, the host
            queues the n calls behind them, and the events bracket only the calls."""
            for _ in range(2):
                fn()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            for _ in range(6):
                big @ big
            e0.record()
            for _ in range(n):
                fn()
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) / n * 1e3
        us = device_us(decode_step)
        us1 = device_us(lambda: decode_step(1))
        import time as _time
        torch.cuda.synchronize()
        t0 = _time.perf_counter()
        for _ in range(20):
            decode_step()
        torch.cuda.synchronize()
        wall_us = (_time.perf_counter() - t0) / 20 * 1e6
        # the same step as one CUDA graph (fill count in device memory): wall time per replayed step
        cache._set_length(Tk - 1)
        dec = nsa.GraphedDecoder(cache, H)
        dec.q.copy_(q1); dec.k.copy_(k1); dec.v.copy_(k1); dec.gate_logits.copy_(g1)
        for _ in range(5):
            dec.step()
        torch.cuda.synchronize()
        t0 = _time.perf_counter()
        for _ in range(100):
            dec.step()
        torch.cuda.synchronize()
        graph_us = (_time.perf_counter() - t0) / 100 * 1e6
        ops.device_status()
        del big, dec
        print(json.dumps({"metric": "nsa_decode_step_us", "value": us, "unsplit_launch_us": us1, "wall_us_python_host": wall_us,
                          "wall_us_cuda_graph": graph_us, "tokens_per_s_cuda_graph": B / (graph_us * 1e-6),
                          "tokens_per_s": B / (us * 1e-6),
                          "config": {"workload": f"decode 1 token/sequence, B={B} cached={Tk} Hq={H} Hkv={Hkv} D={D} bf16, "
                                                 f"cmp={b.cmp_block}/{b.cmp_stride} top-{b.top_k} W={b.window}"}}), flush=True)
        del cache
        torch.cuda.empty_cache()


def run_reference_protocol(a):
    """The reference's measurement protocol (nsa/bench/throughput.py:28-48 and its multi-seed pooling): for each of
    seeds 0, 1, 2: 25 warm-up iterations, 100 timed ones with a CUDA-event pair and a synchronize each; the 300
    samples are pooled; mean and the 95 % percentile bootstrap of the mean (10000 resamples, generator seed 12345)."""
    import numpy as np
    import nsa_from_scratch_b200 as nsa
    torch.cuda.set_device(0)
    cfg = nsa.NSAConfig(block_size_c=a.cmp_block, stride_c=a.cmp_stride, top_k=a.top_k, window_size=a.window, force_first=1,
                        force_local=2, select_per_group=a.select == "group")
    samples = []
    for seed in (0, 1, 2):
        Q, K, V, G = (t.cuda() for t in make_inputs(a, seed))
        for _ in range(25):
            nsa.nsa_forward(Q, K, V, cfg, gate_logits=G)
        torch.cuda.synchronize()
        for _ in range(100):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            nsa.nsa_forward(Q, K, V, cfg, gate_logits=G)
            e1.record()
            torch.cuda.synchronize()
            samples.append(e0.elapsed_time(e1))
        del Q, K, V, G
        torch.cuda.empty_cache()
    x = np.asarray(samples)
    rng = np.random.default_rng(12345)
    means = x[rng.integers(0, len(x), size=(10000, len(x)))].mean(axis=1)
    lo, hi = np.percentile(means, [2.5, 97.5])
    print(json.dumps({"metric": METRIC, "value": a.seq_len / (x.mean() * 1e-3), "unit": UNIT, "ms_per_step": float(x.mean()),
                      "ms_ci95": [float(lo), float(hi)], "tokens_per_s_ci95": [a.seq_len / (hi * 1e-3), a.seq_len / (lo * 1e-3)],
                      "samples": len(x), "protocol": "25 warm-up + 100 iterations x seeds 0,1,2; pooled mean, percentile bootstrap",
                      "config": {"workload": workload_name(a)}}), flush=True)


def main():
    a = parse()
    if a.protocol == "reference" and a.impl == "ours":
        return run_reference_protocol(a)
    if a.decode:
        return sweep_decode(a, shapes=((1, 65536),))
    if a.scorer:
        return sweep_scorer(a)
    if a.train:
        return sweep_train(a, T=min(a.seq_len, 32768))
    if a.sweep:
        return run_sweep(a)
    if a.impl == "reference":
        run_reference(a)
    else:
        run_ours(a)


if __name__ == "__main__":
    main()
