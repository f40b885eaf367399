// Selected-branch backward on the 5th-generation tensor cores (tcgen05 + TMEM + TMA), sm_100a.
// No atomics on floating-point data anywhere: every sum is formed in a fixed order, so dQ, dK and dV
// repeat bit for bit.
//
// Two passes over the same pairs (64 query rows of one head) x (one selected 64-key block):
//
//   key-major pass (dK, dV).  An inverted index -- per (batch, KV head, key block) the list of row
//   groups (query head, query block) that selected it -- is built first (a stable counting sort: per-chunk
//   histograms, prefix sums, ordered fill).
//   A thread block owns one key block, or one segment of a long list.  K and V of the block stay in shared
//   memory; the row groups stream by, two at a time (128 rows), through a TMA ring:
//       S  = Q K^T   dP = dO V^T                      (tcgen05.mma, fp32 in TMEM)
//       P  = exp2(S*scale*log2e - lse*log2e)  dS = P (dP - delta) scale   (softmax warps; 16-bit to shared memory)
//       [dV | . ; . | dK] += [P^T ; dS^T] [dO | Q]      (one M=128 MMA per 16 query rows; the off-diagonal quadrants
//                                                      are computed and dropped: the two useful products have M = 64)
//   dV and dK of the block accumulate in TMEM over the whole list (all query heads of the GQA group included)
//   and are written once.  Segments of a long list leave partial sums that a small kernel adds in segment order.
//
//   query-major pass (dQ).  A thread block owns 128 query rows: two heads of a GQA group that share a block
//   list (64 rows of one head when every head has its own list).  Q and dO stay in shared memory, the listed
//   K/V blocks stream by:  S, dP, dS as above, then dQ += dS K (A = dS from shared memory, B = K MN-major).
//
// Warp roles (18 warps at 112 registers):
//   warp 0  TMA producer      warp 1  MMA issuer (issues whatever is ready: S/dP of a later step or an accumulate)
//   warps 2-9 and 10-17: two softmax groups that alternate steps.  A row of the 128-row tile (= TMEM lane) is
//   shared by two threads, 32 of its 64 columns each -- the log-sum-exp is an input, so the halves of a row need
//   nothing from each other -- which puts four softmax warps on every scheduler to hide each other's waits.
// TMEM columns: S/dP of step parity 0 at [0,64)/[64,128), of parity 1 at [128,192)/[192,256), accumulator from 256.
// Every mbarrier wait is bounded; a wait that gives up raises a block-wide abort flag, the block drains its
// copies (bounded), frees its TMEM, and the status word reports it.
#include "common.cuh"
#include "tc5_ptx.cuh"

#include <cudaTypedefs.h>
#include <type_traits>

namespace nsa {

using namespace tc5;

int make_map(CUtensorMap* m, const void* ptr, long long slabs, long long rows, int D, int dtype);   // attn_fwd_tc5.cu

__device__ int g_bw5_status;   // 0 ok; otherwise (1 + id of the barrier a wait gave up on)

constexpr int BW5_THREADS = 576;      // 18 warps: TMA producer, MMA issuer, 2 softmax groups of 8 warps
constexpr int BW5_MAX_SEL = 256;      // listed blocks per query block (query-major pass)
constexpr int BW5_QB_BITS = 20;       // row group = (head within the group << 20) | query block

struct Bw5Params {
  CUtensorMap tmQ, tmdO, tmK, tmV;
  nsa_bwd_args a;
  float scale_log2;
  int nkb;                 // key blocks
  int G;                   // query heads per KV head
  int shared;              // one block list per KV head (1) or per query head (0)
  // key-major pass
  const int4* items;       // [owners][capW]: (key block, first row group, row groups, partial slot or -1)
  const int* n_items;      // [owners]
  int capW;
  const uint32_t* rg_list; // [owners][cap_rg]
  long long cap_rg;
  float* partials;         // [owners][capP][2][64][D]
  int capP;
  // query-major pass
  int NG;                  // row groups (heads) per tile: 2 or 1
  int NGT;                 // tiles per (batch, KV head, query block)
};

// barrier ids (the ring of streamed tiles has up to 8 stages)
enum { BW_RES = 0, BW_STFULL = 1, BW_STEMPTY = 9, BW_SFULL = 17, BW_SFREE = 19, BW_PFULL = 21, BW_PEMPTY = 23, BW_ACC = 25, BW_QTMEM = 26, BW_COUNT = 27 };

// Stages of the ring of streamed tiles.  A stage is held from the issue of its copy until the accumulate MMA of its step
// has read it, i.e. across the whole softmax of the step, so the ring is as deep as shared memory allows: key-major
// 4 x 32 KB at D=64 and 2 x 64 KB at D=128, query-major 8 x 16 KB at D=64 and 4 x 32 KB at D=128.
__host__ __device__ constexpr int bw5_stages(int D, int mode) { return mode == 0 ? (D == 64 ? 4 : 2) : (D == 64 ? 8 : 4); }

__device__ __forceinline__ bool bw5_legal(int blk, int qb, int nkb, int Tq, int offset, int causal) {
  if (blk < 0 || blk >= nkb) return false;
  if (!causal) return true;
  const int last_pos = min(qb * 64 + 64, Tq) - 1 + offset;
  return (long long)blk * 64 <= (long long)last_pos;
}

// MODE 0: key-major pass (dK, dV).  MODE 1: query-major pass (dQ).
template <int D, int FMT, int MODE>
__global__ void __launch_bounds__(BW5_THREADS, 1) nsa_bwd_tc5_kernel(const __grid_constant__ Bw5Params p) {
  using T = typename std::conditional<FMT == 1, __nv_bfloat16, __half>::type;
  constexpr int DH = D / 64;                    // 64-element (128-byte) halves of a row
  constexpr int T128 = DH * 128 * 128;          // bytes of a 128-row tile (halves 16384 bytes apart)
  constexpr int T64 = DH * 64 * 128;            // bytes of a 64-row tile (halves 8192 bytes apart)
  constexpr int RES_BYTES = MODE == 0 ? 2 * T64 : 2 * T128;   // resident: K,V (key-major) or Q,dO (query-major)
  constexpr int ST_BYTES = MODE == 0 ? 2 * T128 : 2 * T64;    // one ring stage: dO,Q (key-major) or K,V (query-major)
  constexpr int PB_BYTES = MODE == 0 ? 32768 : 16384;         // one P|dS buffer (key-major) or dS buffer (query-major)
  constexpr int NST = bw5_stages(D, MODE);
  // Query-major pass: the A operands that change slowly or are made by the softmax threads live in TMEM instead of shared
  // memory -- the MMAs of a step then read only their B operands (K, V tiles) from shared memory, whose bandwidth is what
  // bounds these small (N = 64) MMAs.  dS (16-bit, 32 columns per buffer) always; Q and dO (32 columns each) at D=64,
  // where the columns are there: S/dP [0,256)  dQ [256,256+D)  dS [384,448)  Q [448,480)  dO [480,512).
  constexpr bool DS_TMEM = MODE == 1;
  constexpr bool Q_TMEM = MODE == 1 && D == 64;
  const nsa_bwd_args& a = p.a;

  // ---- work item (uniform over the block; blocks beyond the item count leave before anything is set up) ----
  const int NL = a.B * a.Hkv;
  int owner, b, hk, c = 0, n_rg = 0, slot = -1, qb = 0, h0 = 0, ng = 0;
  const uint32_t* rgl = nullptr;
  if constexpr (MODE == 0) {
    owner = (int)(blockIdx.x % (unsigned)NL);
    const int ii = (int)(blockIdx.x / (unsigned)NL);
    if (ii >= p.n_items[owner]) return;
    const int4 item = p.items[(size_t)owner * p.capW + ii];
    c = item.x; n_rg = item.z; slot = item.w;
    rgl = p.rg_list + (size_t)owner * p.cap_rg + item.y;
  } else {
    const int per_qb = NL * p.NGT;
    qb = a.nq - 1 - (int)(blockIdx.x / (unsigned)per_qb);
    const int rem = (int)(blockIdx.x % (unsigned)per_qb);
    owner = rem / p.NGT;
    const int ht = rem % p.NGT;
    h0 = ht * p.NG;
    ng = min(p.NG, p.G - h0);
  }
  b = owner / a.Hkv;
  hk = owner % a.Hkv;
  const int kv_slab = owner;

  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sRes = smem_u32(smem);
  const uint32_t sSt = sRes + RES_BYTES;
  unsigned char* pb_ptr = smem + RES_BYTES + NST * ST_BYTES;
  const uint32_t sPb = smem_u32(pb_ptr);
  __shared__ __align__(8) uint64_t bars[BW_COUNT];
  __shared__ int sel_list[BW5_MAX_SEL];
  __shared__ int sel_n;
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_flag;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  auto bar = [&](int id) { return smem_u32(&bars[id]); };

  if (tid == 0) {
    abort_flag = 0;
    for (int i = 0; i < BW_COUNT; ++i)
      mbar_init(bar(i), (i == BW_SFREE || i == BW_SFREE + 1 || i == BW_PFULL || i == BW_PFULL + 1) ? 256 : (i == BW_QTMEM ? 512 : 1));
    fence_barrier_init();
  }
  if (warp == 1) { tmem_alloc(smem_u32(&tmem_base_s), 512); tmem_relinquish(); }
  if (MODE == 1 && warp == 2) {
    // the key blocks this query block lists, in list order, illegal slots dropped
    const int hi_ = p.shared ? hk : hk * p.G + h0;
    const int32_t* row = a.idx + (((size_t)b * a.Hi + hi_) * a.nq + qb) * a.top_k;
    int n = 0;
    for (int s0 = 0; s0 < a.top_k; s0 += 32) {
      const int s = s0 + lane;
      const int blk = s < a.top_k ? row[s] : -1;
      const bool ok = bw5_legal(blk, qb, p.nkb, a.Tq, a.offset, a.causal);
      const unsigned m = __ballot_sync(0xffffffffu, ok);
      if (ok) sel_list[n + __popc(m & ((1u << lane) - 1))] = blk;
      n += __popc(m);
    }
    if (lane == 0) sel_n = n;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_s;
  const int nsteps = MODE == 0 ? (n_rg + 1) >> 1 : sel_n;

  // row group g (0 or 1) of step `st`: head within the KV group and query block; valid == false: rows are zero
  auto row_group = [&](int st, int g, int& hl, int& qblk) -> bool {
    if constexpr (MODE == 0) {
      const int e = 2 * st + g;
      if (e >= n_rg) { hl = 0; qblk = 0; return false; }
      const uint32_t v = rgl[e];
      hl = (int)(v >> BW5_QB_BITS); qblk = (int)(v & ((1u << BW5_QB_BITS) - 1));
      return true;
    } else {
      hl = h0 + g; qblk = qb;
      return g < ng;
    }
  };
  const int oob_row = (a.Tq + 63) / 64 * 64;    // a box that starts here lies outside the tensor: TMA fills it with zeros

  int fail_id = 0;
  int last_st = -1;        // producer: last step whose copies were issued

  if (warp == 0) {
    // =============================== TMA producer ===============================
    const bool leader = elect_one();
    if (leader) {
      tma_prefetch_desc(&p.tmQ); tma_prefetch_desc(&p.tmdO); tma_prefetch_desc(&p.tmK); tma_prefetch_desc(&p.tmV);
      mbar_expect_tx(bar(BW_RES), RES_BYTES);
      if constexpr (MODE == 0) {
        for (int dh = 0; dh < DH; ++dh) {
          tma_load_3d(sRes + dh * 8192, &p.tmK, bar(BW_RES), dh * 64, c * 64, kv_slab);
          tma_load_3d(sRes + T64 + dh * 8192, &p.tmV, bar(BW_RES), dh * 64, c * 64, kv_slab);
        }
      } else {
        for (int g = 0; g < 2; ++g) {
          int hl, qblk;
          const bool ok = row_group(0, g, hl, qblk);
          const int slab = ok ? b * a.H + hk * p.G + hl : 0, row = ok ? qblk * 64 : oob_row;
          for (int dh = 0; dh < DH; ++dh) {
            tma_load_3d(sRes + dh * 16384 + g * 8192, &p.tmQ, bar(BW_RES), dh * 64, row, slab);
            tma_load_3d(sRes + T128 + dh * 16384 + g * 8192, &p.tmdO, bar(BW_RES), dh * 64, row, slab);
          }
        }
      }
    }
    __syncwarp();
    // Key-major: the streamed Q/dO tiles come from HBM (each is read by few thread blocks), about 1800 clocks per copy,
    // more than the ring hides; the tiles of step st+PF are therefore pulled into L2 ahead of their copy.
    constexpr int PF = NST + 3;
    auto prefetch_step = [&](int st) {
      if constexpr (MODE == 0) {
        if (st < nsteps) {
          for (int g = 0; g < 2; ++g) {
            int hl, qblk;
            if (!row_group(st, g, hl, qblk)) continue;
            if (leader) {
              const int slab = b * a.H + hk * p.G + hl;
              for (int dh = 0; dh < DH; ++dh) {
                tma_prefetch_3d(&p.tmdO, dh * 64, qblk * 64, slab);
                tma_prefetch_3d(&p.tmQ, dh * 64, qblk * 64, slab);
              }
            }
          }
        }
      }
    };
    for (int st = NST; st < PF; ++st) prefetch_step(st);
    bool ok = true;
    for (int st = 0; st < nsteps && ok; ++st) {
      const int s = st % NST;
      prefetch_step(st + PF);
      ok = __all_sync(0xffffffffu, mbar_wait(bar(BW_STEMPTY + s), ((st / NST) & 1) ^ 1, &abort_flag));
      if (!ok) { fail_id = BW_STEMPTY + s + 1; break; }
      const uint32_t dst = sSt + s * ST_BYTES;
      if constexpr (MODE == 0) {
        int hl[2], qblk[2];
        bool okg[2];
        for (int g = 0; g < 2; ++g) okg[g] = row_group(st, g, hl[g], qblk[g]);
        if (leader) {
          mbar_expect_tx(bar(BW_STFULL + s), ST_BYTES);
          for (int g = 0; g < 2; ++g) {
            const int slab = okg[g] ? b * a.H + hk * p.G + hl[g] : 0, row = okg[g] ? qblk[g] * 64 : oob_row;
            for (int dh = 0; dh < DH; ++dh) {
              tma_load_3d(dst + dh * 16384 + g * 8192, &p.tmdO, bar(BW_STFULL + s), dh * 64, row, slab);
              tma_load_3d(dst + T128 + dh * 16384 + g * 8192, &p.tmQ, bar(BW_STFULL + s), dh * 64, row, slab);
            }
          }
        }
      } else {
        const int blk = sel_list[st];
        if (leader) {
          mbar_expect_tx(bar(BW_STFULL + s), ST_BYTES);
          for (int dh = 0; dh < DH; ++dh) {
            tma_load_3d(dst + dh * 8192, &p.tmK, bar(BW_STFULL + s), dh * 64, blk * 64, kv_slab);
            tma_load_3d(dst + T64 + dh * 8192, &p.tmV, bar(BW_STFULL + s), dh * 64, blk * 64, kv_slab);
          }
        }
      }
      last_st = st;
      __syncwarp();
    }
  } else if (warp == 1) {
    // =============================== MMA issuer ===============================
    const bool leader = elect_one();
    constexpr uint32_t IDESC_S = idesc_f16(FMT, 128, 64, 0, 0);            // [128 rows x 64 keys] = A(K-major) B(K-major)^T
    constexpr uint32_t IDESC_ACC = MODE == 0 ? idesc_f16(FMT, 128, 2 * D, 1, 1)   // [P^T;dS^T] (MN-major) x [dO|Q] (MN-major)
                                             : idesc_f16(FMT, 128, D, 0, 1);      // dS (K-major) x K (MN-major)
    bool ok = __all_sync(0xffffffffu, mbar_wait(bar(BW_RES), 0, &abort_flag));
    if (!ok) fail_id = BW_RES + 1;
    // byte offsets of the 16-element k-step `ks` in a 128-row (A side) and a 64-row (B side) K-major tile
    auto offA = [](int ks) { return (uint32_t)(((ks >> 2) * 16384 + (ks & 3) * 32) >> 4); };
    auto offB = [](int ks) { return (uint32_t)(((ks >> 2) * 8192 + (ks & 3) * 32) >> 4); };
    const uint32_t tACC = tmem + 256;
    if constexpr (Q_TMEM) {
      if (ok) {
        ok = __all_sync(0xffffffffu, mbar_wait(bar(BW_QTMEM), 0, &abort_flag));
        if (!ok) fail_id = BW_QTMEM + 1;
        tc_fence_after();
      }
    }

    // S = Q K^T and dP = dO V^T of step st into the TMEM buffer of its parity
    auto issue_sdp = [&](int st) {
      const int s = st % NST, sb = st & 1;
      tc_fence_after();
      if (leader) {
        const uint32_t st_base = sSt + s * ST_BYTES;
        // key-major: A = streamed Q / dO, B = resident K / V;  query-major: A = resident Q / dO, B = streamed K / V
        const uint64_t aS = smem_desc_sw128(MODE == 0 ? st_base + T128 : sRes, 16, 1024);
        const uint64_t aP = smem_desc_sw128(MODE == 0 ? st_base : sRes + T128, 16, 1024);
        const uint64_t bS = smem_desc_sw128(MODE == 0 ? sRes : st_base, 16, 1024);
        const uint64_t bP = smem_desc_sw128(MODE == 0 ? sRes + T64 : st_base + T64, 16, 1024);
        const uint32_t tS = tmem + sb * 128, tdP = tS + 64;
        if constexpr (Q_TMEM) {
#pragma unroll
          for (int ks = 0; ks < D / 16; ++ks) mma_ts(tS, tmem + 448 + ks * 8, bS + offB(ks), IDESC_S, ks == 0 ? 0u : 1u);
#pragma unroll
          for (int ks = 0; ks < D / 16; ++ks) mma_ts(tdP, tmem + 480 + ks * 8, bP + offB(ks), IDESC_S, ks == 0 ? 0u : 1u);
        } else {
#pragma unroll
          for (int ks = 0; ks < D / 16; ++ks) mma_ss(tS, aS + offA(ks), bS + offB(ks), IDESC_S, ks == 0 ? 0u : 1u);
#pragma unroll
          for (int ks = 0; ks < D / 16; ++ks) mma_ss(tdP, aP + offA(ks), bP + offB(ks), IDESC_S, ks == 0 ? 0u : 1u);
        }
        tc_commit(bar(BW_SFULL + sb));
      }
      __syncwarp();
    };
    // the accumulate MMA of step st (reads P/dS of its parity and ring stage st % NST; frees both)
    auto issue_acc = [&](int st) {
      const int s = st % NST, sb = st & 1;
      tc_fence_after();
      if (leader) {
        const uint32_t st_base = sSt + s * ST_BYTES, pbuf = sPb + sb * PB_BYTES;
        if constexpr (MODE == 0) {
          // A: [P^T ; dS^T]: M = 64 keys of P then 64 keys of dS (chunks 16384 bytes apart), K = 128 query rows
          // B: [dO | Q]: N = 2*D in 64-element chunks 16384 bytes apart, K = the same 128 query rows
          const uint64_t dA = smem_desc_sw128(pbuf, 16384, 1024);
          const uint64_t dB = smem_desc_sw128(st_base, 16384, 1024);
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) mma_ss(tACC, dA + kk * 128, dB + kk * 128, IDESC_ACC, (st > 0 || kk > 0) ? 1u : 0u);
        } else {
          // A: dS [128 rows x 64 keys] from TMEM (16-bit pairs, 8 columns per 16 keys);  B: K [64 keys x D] MN-major (halves 8192 bytes apart)
          const uint64_t dB = smem_desc_sw128(st_base, 8192, 1024);
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) mma_ts(tACC, tmem + 384 + sb * 32 + ks * 8, dB + ks * 128, IDESC_ACC, (st > 0 || ks > 0) ? 1u : 0u);
          (void)pbuf;
        }
        tc_commit(bar(BW_PEMPTY + sb));
        tc_commit(bar(BW_STEMPTY + s));
      }
      __syncwarp();
    };
    // Whatever is ready is issued: S/dP of step ns as soon as its tiles have landed and the softmax group of its
    // parity holds the previous S/dP of that buffer in registers; the accumulate of step na as soon as its P/dS are in
    // shared memory.  (A fixed order makes one of the two softmax groups wait for the other through this warp.)
    int ns = 0, na = 0;
    long long idle = 0;
    while (na < nsteps && ok) {
      bool did = false;
      if (ns < nsteps) {
        const bool rdy = mbar_test_wait(bar(BW_STFULL + ns % NST), (ns / NST) & 1) && mbar_test_wait(bar(BW_SFREE + (ns & 1)), ((ns >> 1) & 1) ^ 1);
        if (__all_sync(0xffffffffu, rdy)) { issue_sdp(ns); ++ns; did = true; }
      }
      if (na < ns) {
        const bool rdy = mbar_test_wait(bar(BW_PFULL + (na & 1)), (na >> 1) & 1);
        if (__all_sync(0xffffffffu, rdy)) { issue_acc(na); ++na; did = true; }
      }
      if (did) { idle = 0; continue; }
      ++idle;                                                // bounded: about a second, or until another warp gives up
      __nanosleep(20);                                       // leave the issue slots to the softmax warps of this scheduler
      if (idle > 65536) {
        if (abort_flag || idle > (1 << 23)) { abort_flag = 1; fail_id = (na < ns ? BW_PFULL + (na & 1) : BW_STFULL + ns % NST) + 1; ok = false; break; }
        __nanosleep(100);
      }
    }
    if (ok && nsteps > 0) {
      if (leader) tc_commit(bar(BW_ACC));
      __syncwarp();
    }
  } else {
    // =============================== softmax / epilogue ===============================
    const int grp = (warp - 2) >> 3;                       // handles the steps of parity grp
    const int quarter = warp & 3;                          // the TMEM lanes a warp may touch: 32*(warp % 4) ..
    const int hf = ((warp - 2) >> 2) & 1;                  // which 32 of the row's 64 columns
    const int r = quarter * 32 + lane;                     // row of the 128-row tile == TMEM lane
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const int g2 = r >> 6;
    const uint32_t tS = tmem + lane_addr + grp * 128 + hf * 32, tdP = tS + 64;
    unsigned char* prow = pb_ptr + grp * PB_BYTES + r * 128;           // this row of P (key-major) / dS (query-major)
    const float sc = a.scale;

    // What a query row needs: its log-sum-exp (log2 units), delta*scale, and the last key position it may see.
    // Query-major: the row is fixed.  Key-major: the rows change every step and come through two dependent loads
    // (list entry, then lse/delta), a couple of thousand clocks when taken in line -- so they are fetched ahead: in
    // the iteration of step st the loads of lse/delta for step st+2 (this group's next) and of the list entry for
    // step st+4 are issued, and their results are first touched one iteration later.
    float lse2 = 0.f, dls = 0.f;
    int hi = -1;
    auto entry = [&](int st) -> uint32_t {                   // list entry of this thread's row group at step st, or ~0
      if constexpr (MODE == 0) { const int e = 2 * st + g2; return e < n_rg ? rgl[e] : 0xffffffffu; }
      else return g2 < ng ? (((uint32_t)(h0 + g2) << BW5_QB_BITS) | (uint32_t)qb) : 0xffffffffu;   // the same rows at every step
    };
    struct RowRaw { float l, d; int qi; bool ok; };
    auto fetch = [&](uint32_t ent) -> RowRaw {               // issues the loads (unconditionally, from a safe address, so that
      RowRaw rr;                                             // nothing has to wait for them before `adopt`)
      const int hl = (int)(ent >> BW5_QB_BITS), qblk = (int)(ent & ((1u << BW5_QB_BITS) - 1));
      rr.qi = qblk * 64 + (r & 63);
      rr.ok = ent != 0xffffffffu && rr.qi < a.Tq;
      const size_t ri = rr.ok ? ((size_t)b * a.H + hk * p.G + hl) * a.Tq + rr.qi : 0;
      rr.l = a.lse[ri];
      rr.d = a.delta[ri];
      return rr;
    };
    auto adopt = [&](const RowRaw& rr) {
      lse2 = 0.f; dls = 0.f; hi = -1;
      if (rr.ok && rr.l > -INFINITY) {
        lse2 = rr.l * kLog2e;
        dls = rr.d * sc;
        hi = a.causal ? min(rr.qi + a.offset, a.sel_key_limit - 1) : a.sel_key_limit - 1;
      }
    };
    bool ok = true;
    if constexpr (Q_TMEM) {
      // Q (softmax group 0) and dO (group 1) from their swizzled shared-memory tiles into TMEM: a thread moves its 64
      // bytes of its row (32 elements = 16 columns of 16-bit pairs)
      ok = __all_sync(0xffffffffu, mbar_wait(bar(BW_RES), 0, &abort_flag));
      if (!ok) fail_id = BW_RES + 1;
      if (ok) {
        const unsigned char* src = smem + grp * T128 + r * 128;
        uint32_t w[16];
#pragma unroll
        for (int c4 = 0; c4 < 4; ++c4) {
          const uint4 v = *reinterpret_cast<const uint4*>(src + (((hf * 4 + c4) ^ (r & 7)) << 4));
          w[4 * c4] = v.x; w[4 * c4 + 1] = v.y; w[4 * c4 + 2] = v.z; w[4 * c4 + 3] = v.w;
        }
        tmem_st16(tmem + lane_addr + 448 + grp * 32 + hf * 16, w);
        tc_wait_st();
        tc_fence_before();
        mbar_arrive(bar(BW_QTMEM));
      }
    }
    RowRaw nxt = fetch(entry(grp));                          // rows of this group's first step
    uint32_t ent_nn = MODE == 0 ? entry(grp + 2) : 0xffffffffu;

#pragma unroll 1
    for (int st = grp; st < nsteps && ok; st += 2) {
      const int ph = (st >> 1) & 1;
      int j0;
      if constexpr (MODE == 0) {
        adopt(nxt);
        nxt = fetch(ent_nn);
        ent_nn = entry(st + 4);
        j0 = c * 64;
      } else {
        if (st == grp) adopt(nxt);
        j0 = sel_list[st] * 64;
      }
      const int vhi = min(hi, min(j0 + 64, a.sel_key_limit) - 1) - j0;   // columns 0..vhi of the tile count for this row
      ok = __all_sync(0xffffffffu, mbar_wait(bar(BW_SFULL + grp), ph, &abort_flag));
      if (!ok) { fail_id = BW_SFULL + grp + 1; break; }
      tc_fence_after();
      uint32_t sv[32], dv[32];
      tmem_ld32(tS, sv);
      tmem_ld32(tdP, dv);
      tc_wait_ld();
      tc_fence_before();
      mbar_arrive(bar(BW_SFREE + grp));                    // S and dP are in registers: the next step may overwrite them
      // P and dS, packed to 16 bits.  Only tiles on the causal diagonal (or with rows that take no part) need the
      // per-element mask; the other tiles of a warp skip its compare and select.
      uint32_t pk[16], dk[16];
      auto compute = [&](auto masked) {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float p0 = ex2(fmaf(__uint_as_float(sv[2 * i]), p.scale_log2, -lse2));
          float p1 = ex2(fmaf(__uint_as_float(sv[2 * i + 1]), p.scale_log2, -lse2));
          if constexpr (decltype(masked)::value) {
            if (hf * 32 + 2 * i > vhi) p0 = 0.f;
            if (hf * 32 + 2 * i + 1 > vhi) p1 = 0.f;
          }
          const float d0 = p0 * fmaf(__uint_as_float(dv[2 * i]), sc, -dls);
          const float d1 = p1 * fmaf(__uint_as_float(dv[2 * i + 1]), sc, -dls);
          pk[i] = Elem<T>::pack(p0, p1);
          dk[i] = Elem<T>::pack(d0, d1);
        }
      };
      if (__all_sync(0xffffffffu, vhi >= 63)) compute(std::false_type{});
      else compute(std::true_type{});
      ok = __all_sync(0xffffffffu, mbar_wait(bar(BW_PEMPTY + grp), ph ^ 1, &abort_flag));
      if (!ok) { fail_id = BW_PEMPTY + grp + 1; break; }
      if constexpr (DS_TMEM) {
        // dS as the accumulate MMA's A operand in TMEM: 16 columns of 16-bit pairs for this thread's 32 keys
        tmem_st16(tmem + lane_addr + 384 + grp * 32 + hf * 16, dk);
        tc_wait_st();
        tc_fence_before();
      } else {
        // this thread's 64 bytes of the 128-byte row; 16-byte chunks XOR-swizzled with the row (the layout TMA's 128-byte swizzle gives)
#pragma unroll
        for (int c4 = 0; c4 < 4; ++c4) {
          const int ch = hf * 4 + c4, i = c4 * 4;
          const uint32_t sw = (uint32_t)((ch ^ (r & 7)) << 4);
          *reinterpret_cast<uint4*>(prow + sw) = make_uint4(pk[i], pk[i + 1], pk[i + 2], pk[i + 3]);
          *reinterpret_cast<uint4*>(prow + 16384 + sw) = make_uint4(dk[i], dk[i + 1], dk[i + 2], dk[i + 3]);
        }
        fence_proxy_async();
      }
      mbar_arrive(bar(BW_PFULL + grp));
    }

    // ---- epilogue: the accumulator is complete once the last MMA has landed ----
    if (ok && nsteps > 0) {
      ok = __all_sync(0xffffffffu, mbar_wait(bar(BW_ACC), 0, &abort_flag));
      if (!ok) fail_id = BW_ACC + 1;
      tc_fence_after();
    }
    if (ok) {
      constexpr int HC = D / 4;                            // the four warps that share a lane quarter split the columns
      const int part = grp * 2 + hf;
      auto load_part = [&](uint32_t taddr, uint32_t (&v)[HC]) {
        if constexpr (HC == 32) tmem_ld32(taddr, v);
        else tmem_ld16(taddr, v);
        tc_wait_ld();
      };
      if constexpr (MODE == 0) {
        // lanes 0-63: dV of key (lane), columns [0,D);  lanes 64-127: dK of key (lane-64), columns [D,2D)
        const int which = g2, kr = r & 63;
        const int key = c * 64 + kr;
        float* dst;
        const bool direct = slot < 0;
        if (direct) dst = (which ? a.dK_f : a.dV_f) + ((size_t)kv_slab * a.Tk + key) * D + part * HC;
        else dst = p.partials + ((((size_t)owner * p.capP + slot) * 2 + which) * 64 + kr) * D + part * HC;
        const bool wr = !direct || key < a.Tk;
        uint32_t v[HC];
        load_part(tmem + lane_addr + 256 + which * D + part * HC, v);
        if (wr) {
#pragma unroll
          for (int q4 = 0; q4 < HC / 4; ++q4) {
            float4 o = make_float4(__uint_as_float(v[4 * q4]), __uint_as_float(v[4 * q4 + 1]), __uint_as_float(v[4 * q4 + 2]),
                                   __uint_as_float(v[4 * q4 + 3]));
            float4* dp4 = reinterpret_cast<float4*>(dst) + q4;
            if (direct) { const float4 old = *dp4; o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w; }
            *dp4 = o;
          }
        }
      } else {
        const uint32_t ent = entry(0);
        const int hl = (int)(ent >> BW5_QB_BITS);
        const int qi = qb * 64 + (r & 63);
        const bool wr = ent != 0xffffffffu && qi < a.Tq;
        const size_t base = (((size_t)b * a.H + hk * p.G + hl) * a.Tq + qi) * D + part * HC;
        uint32_t v[HC];
        if (nsteps > 0) load_part(tmem + lane_addr + 256 + part * HC, v);
        else {
#pragma unroll
          for (int i = 0; i < HC; ++i) v[i] = 0u;
        }
        if (wr) {
          if (a.dq_dtype == NSA_FP32) {
            float4* dp4 = reinterpret_cast<float4*>(reinterpret_cast<float*>(a.dQ) + base);
#pragma unroll
            for (int q4 = 0; q4 < HC / 4; ++q4)
              dp4[q4] = make_float4(__uint_as_float(v[4 * q4]), __uint_as_float(v[4 * q4 + 1]), __uint_as_float(v[4 * q4 + 2]),
                                    __uint_as_float(v[4 * q4 + 3]));
          } else {
            uint4* dp4 = reinterpret_cast<uint4*>(reinterpret_cast<T*>(a.dQ) + base);
#pragma unroll
            for (int q4 = 0; q4 < HC / 8; ++q4)
              dp4[q4] = make_uint4(Elem<T>::pack(__uint_as_float(v[8 * q4]), __uint_as_float(v[8 * q4 + 1])),
                                   Elem<T>::pack(__uint_as_float(v[8 * q4 + 2]), __uint_as_float(v[8 * q4 + 3])),
                                   Elem<T>::pack(__uint_as_float(v[8 * q4 + 4]), __uint_as_float(v[8 * q4 + 5])),
                                   Elem<T>::pack(__uint_as_float(v[8 * q4 + 6]), __uint_as_float(v[8 * q4 + 7])));
          }
        }
      }
    }
  }

  // ---- teardown (every path reaches it) ----
  if (fail_id != 0) atomicCAS(&g_bw5_status, 0, fail_id);
  tc_fence_before();
  __syncthreads();
  if (abort_flag && warp == 0 && lane == 0) {
    // let copies already in flight land (bounded) before the block's shared memory is handed back
    for (int i = 0; i < 20000 && !mbar_try_wait(bar(BW_RES), 0); ++i) __nanosleep(100);
    for (int k = 0; k < NST && last_st - k >= 0; ++k) {
      const int st = last_st - k;
      for (int i = 0; i < 20000 && !mbar_try_wait(bar(BW_STFULL + st % NST), (st / NST) & 1); ++i) __nanosleep(100);
    }
  }
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, 512); }
}

// ---------------------------------------------------------------- inverted index
// A stable counting sort of the list entries (list, query block, slot) by key block, in three steps whose work is
// linear in the number of entries: per-chunk histograms, prefix sums over (list, chunk) per key block, ordered fill.
constexpr int BW5_QC = 32;            // query blocks per chunk
constexpr int BW5_MAX_NKB = 12288;    // key blocks a histogram in shared memory can hold

// hist[(list*nchunks + chunk)*nkb + c] = legal entries of the chunk's query blocks that name key block c
__global__ void __launch_bounds__(256) bw5_hist_kernel(const int32_t* __restrict__ idx, int* __restrict__ hist, int nq, int top_k, int nkb,
                                                       int nchunks, int Tq, int offset, int causal) {
  extern __shared__ int h_s[];
  const int chunk = blockIdx.x, list = blockIdx.y;
  for (int i = threadIdx.x; i < nkb; i += blockDim.x) h_s[i] = 0;
  __syncthreads();
  const int qb0 = chunk * BW5_QC, qb1 = min(qb0 + BW5_QC, nq);
  const int32_t* row = idx + (size_t)list * nq * top_k;
  for (int e = qb0 * top_k + threadIdx.x; e < qb1 * top_k; e += blockDim.x) {
    const int blk = row[e];
    if (bw5_legal(blk, e / top_k, nkb, Tq, offset, causal)) atomicAdd(&h_s[blk], 1);
  }
  __syncthreads();
  int* out = hist + ((size_t)list * nchunks + chunk) * nkb;
  for (int i = threadIdx.x; i < nkb; i += blockDim.x) out[i] = h_s[i];
}

// Per (owner, key block c): the histogram entries of the owner's lists, in (list, chunk) order, become exclusive prefix
// sums (the position of the chunk's first entry in c's list); cnt[owner][c] = row groups in the list.  A thread block
// takes 32 key blocks (one per lane); its 8 warps split the (list, chunk) sequence and combine through shared memory.
__global__ void __launch_bounds__(256) bw5_prefix_kernel(int* __restrict__ hist, int* __restrict__ cnt, int nkb, int nchunks, int Hi,
                                                         int Hkv, int G, int shared) {
  __shared__ int part[8][32];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int owner = blockIdx.y, b = owner / Hkv, hk = owner % Hkv;
  const int c = blockIdx.x * 32 + lane;
  const bool in = c < nkb;
  const int nlists = shared ? 1 : G;
  const int nseq = nlists * nchunks;
  const int per = (nseq + 7) / 8;
  const int s0 = min(w * per, nseq), s1 = min(s0 + per, nseq);
  auto at = [&](int s) {
    const int l = s / nchunks, ch = s % nchunks;
    const int list = b * Hi + (shared ? hk : hk * G + l);
    return hist + ((size_t)list * nchunks + ch) * nkb + c;
  };
  int sum = 0;
  for (int sb = s0; sb < s1; sb += 8) {
    int v[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) v[k] = (in && sb + k < s1) ? __ldcg(at(sb + k)) : 0;
#pragma unroll
    for (int k = 0; k < 8; ++k) sum += v[k];
  }
  part[w][lane] = sum;
  __syncthreads();
  int run = 0, total = 0;
#pragma unroll
  for (int k = 0; k < 8; ++k) { if (k < w) run += part[k][lane]; total += part[k][lane]; }
  for (int sb = s0; sb < s1; sb += 8) {
    int v[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) v[k] = (in && sb + k < s1) ? __ldcg(at(sb + k)) : 0;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      if (in && sb + k < s1) __stcg(at(sb + k), run);
      run += v[k];
    }
  }
  if (w == 0 && in) cnt[(size_t)owner * nkb + c] = total * (shared ? G : 1);
}

// Per owner (batch, KV head): exclusive scans over the key blocks of (row groups, segments, partial slots); writes the
// list offsets and the work items of the key-major pass.  One block of 1024 threads per owner.
__global__ void __launch_bounds__(1024) bw5_plan_kernel(const int* __restrict__ cnt, int* __restrict__ off, int2* __restrict__ seginfo,
                                                        int4* __restrict__ items, int* __restrict__ n_items, int nkb, int L, int capW) {
  __shared__ int wsum[3][32];
  __shared__ int run[3];
  const int owner = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid < 3) run[tid] = 0;
  __syncthreads();
  for (int c0 = 0; c0 < nkb; c0 += 1024) {
    const int c = c0 + tid;
    const int n = c < nkb ? cnt[(size_t)owner * nkb + c] : 0;
    const int ns = (n + L - 1) / L;
    const int np = ns >= 2 ? ns : 0;
    int v[3] = {n, ns, np}, inc[3];
#pragma unroll
    for (int k = 0; k < 3; ++k) {
      int x = v[k];
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) { const int y = __shfl_up_sync(0xffffffffu, x, d); if (lane >= d) x += y; }
      inc[k] = x;
      if (lane == 31) wsum[k][warp] = x;
    }
    __syncthreads();
    if (warp == 0) {
#pragma unroll
      for (int k = 0; k < 3; ++k) {
        int x = wsum[k][lane];
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) { const int y = __shfl_up_sync(0xffffffffu, x, d); if (lane >= d) x += y; }
        wsum[k][lane] = x;                                   // inclusive over warps
      }
    }
    __syncthreads();
    int ex[3];
#pragma unroll
    for (int k = 0; k < 3; ++k) ex[k] = run[k] + (warp > 0 ? wsum[k][warp - 1] : 0) + inc[k] - v[k];
    if (c < nkb) {
      off[(size_t)owner * nkb + c] = ex[0];
      seginfo[(size_t)owner * nkb + c] = make_int2(np ? ex[2] : -1, ns);
      for (int s = 0; s < ns; ++s)
        items[(size_t)owner * capW + ex[1] + s] = make_int4(c, ex[0] + s * L, min(L, n - s * L), np ? ex[2] + s : -1);
    }
    __syncthreads();
    if (tid < 3) run[tid] += wsum[tid][31];
    __syncthreads();
  }
  if (tid == 0) n_items[owner] = run[1];
}

// One warp per (list, chunk): walks the chunk's query blocks in order and writes each legal entry at its position in
// the key block's list -- (head, query block, slot) order, so the sums of the key-major pass are formed in a fixed
// order.  hist holds the chunk's starting positions (bw5_prefix_kernel) and serves as the running cursor.
__global__ void __launch_bounds__(256) bw5_fill_kernel(const int32_t* __restrict__ idx, int* __restrict__ hist, const int* __restrict__ off,
                                                       uint32_t* __restrict__ rg_list, long long cap_rg, int n_lists, int Hi, int Hkv, int nq,
                                                       int top_k, int nkb, int nchunks, int Tq, int offset, int causal, int G, int shared) {
  const long long w = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= (long long)n_lists * nchunks) return;
  const int list = (int)(w / nchunks), chunk = (int)(w % nchunks);
  const int b = list / Hi, hi = list % Hi;
  const int hk = hi / (Hi / Hkv), hl = shared ? 0 : hi % G;
  const int owner = b * Hkv + hk;
  int* cur = hist + ((size_t)list * nchunks + chunk) * nkb;
  const int* off_o = off + (size_t)owner * nkb;
  uint32_t* dst = rg_list + (size_t)owner * cap_rg;
  const int32_t* row = idx + (size_t)list * nq * top_k;
  const int qb0 = chunk * BW5_QC, qb1 = min(qb0 + BW5_QC, nq);
  for (int qb = qb0; qb < qb1; ++qb) {
    for (int sl0 = 0; sl0 < top_k; sl0 += 32) {
      const int sl = sl0 + lane;
      const int blk = sl < top_k ? row[(size_t)qb * top_k + sl] : -1;
      const bool ok = bw5_legal(blk, qb, nkb, Tq, offset, causal);
      // lanes that name the same key block (a list may repeat a block) take consecutive positions in slot order
      const unsigned same = __match_any_sync(0xffffffffu, ok ? blk : -1 - lane);
      const int rank = __popc(same & ((1u << lane) - 1));
      int base = 0;
      if (ok) {
        base = __ldcg(cur + blk);
        const int at = base + rank;
        const int o = off_o[blk];
        if (shared) { for (int g = 0; g < G; ++g) dst[(size_t)o + (size_t)at * G + g] = ((uint32_t)g << BW5_QB_BITS) | (uint32_t)qb; }
        else dst[(size_t)o + at] = ((uint32_t)hl << BW5_QB_BITS) | (uint32_t)qb;
      }
      __syncwarp();
      if (ok && rank == 0) __stcg(cur + blk, base + __popc(same));
      __syncwarp();
    }
  }
}

// dK/dV of key blocks whose list was split: the segments' partial sums are added in segment order.
template <int D>
__global__ void __launch_bounds__(256) bw5_reduce_kernel(const float* __restrict__ partials, const int2* __restrict__ seginfo, float* __restrict__ dK,
                                                         float* __restrict__ dV, int nkb, int capP, int Tk) {
  const int owner = blockIdx.y, c = blockIdx.x;
  const int2 si = seginfo[(size_t)owner * nkb + c];
  if (si.x < 0) return;
  constexpr int N4 = 64 * D / 4;
  for (int which = 0; which < 2; ++which) {
    float* out = (which ? dK : dV) + ((size_t)owner * Tk + (size_t)c * 64) * D;
    for (int i = threadIdx.x; i < N4; i += 256) {
      const int key = c * 64 + i / (D / 4);
      if (key >= Tk) continue;
      float4 acc = reinterpret_cast<const float4*>(out)[i];
      for (int s = 0; s < si.y; ++s) {
        const float4 v = reinterpret_cast<const float4*>(partials + (((size_t)owner * capP + si.x + s) * 2 + which) * 64 * D)[i];
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
      }
      reinterpret_cast<float4*>(out)[i] = acc;
    }
  }
}

// ---------------------------------------------------------------- host side
struct Bw5Plan {
  int nkb, G, shared, L, capW, capP, nchunks;
  long long cap_rg, owners, n_lists;
  size_t o_cnt, o_off, o_seg, o_nitems, o_items, o_list, o_hist, o_part, total;
};

bool attention_bwd_tc5_supports(const nsa_bwd_args& a) {
  if (a.branch != NSA_BRANCH_SELECTED) return false;
  if (!(a.dtype == NSA_BF16 || a.dtype == NSA_FP16)) return false;
  if (!(a.D == 64 || a.D == 128)) return false;
  if (a.bm != 64 || a.bn != 64 || a.top_k > BW5_MAX_SEL) return false;
  if (a.nq >= (1 << BW5_QB_BITS) || a.H / a.Hkv >= (1 << (32 - BW5_QB_BITS))) return false;
  if ((a.sel_key_limit + 63) / 64 > BW5_MAX_NKB || (long long)a.B * a.H > 65535) return false;
  if (!(a.scale > 0.f)) return false;
  return true;
}

static Bw5Plan bw5_plan(const nsa_bwd_args& a) {
  Bw5Plan pl;
  pl.nkb = (a.sel_key_limit + 63) / 64;
  pl.G = a.H / a.Hkv;
  pl.shared = a.Hi != a.H ? 1 : 0;
  pl.owners = (long long)a.B * a.Hkv;
  pl.cap_rg = (long long)pl.G * a.nq * a.top_k;
  pl.n_lists = (long long)a.B * a.Hi;
  pl.nchunks = (a.nq + BW5_QC - 1) / BW5_QC;
  // segment length (row groups, even): about 16 work items per SM over the whole launch, between 128 and 1024
  long long L = (pl.cap_rg * pl.owners / 2400 + 1) / 2 * 2;
  pl.L = (int)(L < 128 ? 128 : (L > 1024 ? 1024 : L));
  pl.capW = (int)(pl.nkb + pl.cap_rg / pl.L + 1);
  pl.capP = (int)(2 * pl.cap_rg / pl.L + 2);
  auto up = [](size_t x) { return (x + 255) & ~size_t(255); };
  size_t o = 0;
  pl.o_cnt = o; o = up(o + (size_t)pl.owners * pl.nkb * 4);
  pl.o_nitems = o; o = up(o + (size_t)pl.owners * 4);
  pl.o_off = o; o = up(o + (size_t)pl.owners * pl.nkb * 4);
  pl.o_seg = o; o = up(o + (size_t)pl.owners * pl.nkb * 8);
  pl.o_items = o; o = up(o + (size_t)pl.owners * pl.capW * 16);
  pl.o_list = o; o = up(o + (size_t)pl.owners * pl.cap_rg * 4);
  pl.o_hist = o; o = up(o + (size_t)pl.n_lists * pl.nchunks * pl.nkb * 4);
  pl.o_part = o; o = up(o + (size_t)pl.owners * pl.capP * 2 * 64 * a.D * 4);
  pl.total = o;
  return pl;
}

long long attention_bwd_tc5_scratch_bytes(const nsa_bwd_args& a) { return (long long)bw5_plan(a).total; }

int attention_bwd_tc5(const nsa_bwd_args& a, void* scratch, long long scratch_bytes, cudaStream_t st) {
  const Bw5Plan pl = bw5_plan(a);
  NSA_REQUIRE(scratch != nullptr && scratch_bytes >= (long long)pl.total, NSA_ERR_ARG,
              "selected backward (tcgen05): needs %lld bytes of scratch, %lld given", (long long)pl.total, scratch_bytes);
  NSA_REQUIRE((reinterpret_cast<uintptr_t>(scratch) & 255) == 0, NSA_ERR_ARG, "selected backward (tcgen05): scratch must be 256-byte aligned");
  unsigned char* sc = reinterpret_cast<unsigned char*>(scratch);
  int* cnt = reinterpret_cast<int*>(sc + pl.o_cnt);
  int* n_items = reinterpret_cast<int*>(sc + pl.o_nitems);
  int* off = reinterpret_cast<int*>(sc + pl.o_off);
  int2* seginfo = reinterpret_cast<int2*>(sc + pl.o_seg);
  int4* items = reinterpret_cast<int4*>(sc + pl.o_items);
  uint32_t* rg_list = reinterpret_cast<uint32_t*>(sc + pl.o_list);
  int* hist = reinterpret_cast<int*>(sc + pl.o_hist);
  float* partials = reinterpret_cast<float*>(sc + pl.o_part);

  Bw5Params p;
  p.a = a;
  p.scale_log2 = a.scale * kLog2e;
  p.nkb = pl.nkb; p.G = pl.G; p.shared = pl.shared;
  p.items = items; p.n_items = n_items; p.capW = pl.capW; p.rg_list = rg_list; p.cap_rg = pl.cap_rg;
  p.partials = partials; p.capP = pl.capP;
  p.NG = (pl.shared && pl.G >= 2) ? 2 : 1;
  p.NGT = (pl.G + p.NG - 1) / p.NG;
  int rc;
  if ((rc = make_map(&p.tmQ, a.Q, (long long)a.B * a.H, a.Tq, a.D, a.dtype)) != NSA_OK) return rc;
  if ((rc = make_map(&p.tmdO, a.dO, (long long)a.B * a.H, a.Tq, a.D, a.dtype)) != NSA_OK) return rc;
  if ((rc = make_map(&p.tmK, a.K, (long long)a.B * a.Hkv, a.Tk, a.D, a.dtype)) != NSA_OK) return rc;
  if ((rc = make_map(&p.tmV, a.V, (long long)a.B * a.Hkv, a.Tk, a.D, a.dtype)) != NSA_OK) return rc;

  // inverted index
  NSA_REQUIRE((long long)pl.owners * pl.capW < 2147483647LL && pl.n_lists * pl.nchunks < (1LL << 31) / 32, NSA_ERR_ARG,
              "selected backward: problem too large");
  bw5_hist_kernel<<<dim3((unsigned)pl.nchunks, (unsigned)pl.n_lists), 256, (size_t)pl.nkb * 4, st>>>(a.idx, hist, a.nq, a.top_k, pl.nkb,
                                                                                                  pl.nchunks, a.Tq, a.offset, a.causal);
  bw5_prefix_kernel<<<dim3((unsigned)((pl.nkb + 31) / 32), (unsigned)pl.owners), 256, 0, st>>>(hist, cnt, pl.nkb, pl.nchunks, a.Hi, a.Hkv,
                                                                                             pl.G, pl.shared);
  bw5_plan_kernel<<<(unsigned)pl.owners, 1024, 0, st>>>(cnt, off, seginfo, items, n_items, pl.nkb, pl.L, pl.capW);
  const long long warps = pl.n_lists * pl.nchunks;
  bw5_fill_kernel<<<(unsigned)((warps + 7) / 8), 256, 0, st>>>(a.idx, hist, off, rg_list, pl.cap_rg, (int)pl.n_lists, a.Hi, a.Hkv, a.nq,
                                                              a.top_k, pl.nkb, pl.nchunks, a.Tq, a.offset, a.causal, pl.G, pl.shared);
  if ((rc = launch_status("selected backward index")) != NSA_OK) return rc;

  const int DHh = a.D / 64;
  const size_t smem0 = (size_t)2 * DHh * 64 * 128 + (size_t)bw5_stages(a.D, 0) * 2 * DHh * 128 * 128 + 2 * 32768 + 1024;
  const size_t smem1 = (size_t)2 * DHh * 128 * 128 + (size_t)bw5_stages(a.D, 1) * 2 * DHh * 64 * 128 + 2 * 16384 + 1024;
  const unsigned grid0 = (unsigned)(pl.owners * pl.capW);
  const long long tiles1 = pl.owners * p.NGT * a.nq;
  NSA_REQUIRE(tiles1 < 2147483647LL, NSA_ERR_ARG, "selected backward: %lld query tiles do not fit a grid", tiles1);
#define NSA_BW5_LAUNCH(DD, FF)                                                                                   \
  {                                                                                                               \
    auto f0 = nsa_bwd_tc5_kernel<DD, FF, 0>;                                                                      \
    auto f1 = nsa_bwd_tc5_kernel<DD, FF, 1>;                                                                      \
    NSA_CUDA_OK(cudaFuncSetAttribute(f0, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem0));              \
    NSA_CUDA_OK(cudaFuncSetAttribute(f1, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem1));              \
    f0<<<grid0, BW5_THREADS, smem0, st>>>(p);                                                                     \
    bw5_reduce_kernel<DD><<<dim3((unsigned)pl.nkb, (unsigned)pl.owners), 256, 0, st>>>(partials, seginfo, a.dK_f, a.dV_f, pl.nkb, \
                                                                                       pl.capP, a.Tk);           \
    f1<<<(unsigned)tiles1, BW5_THREADS, smem1, st>>>(p);                                                          \
  }
  const int fmt = a.dtype == NSA_BF16 ? 1 : 0;
  if (a.D == 128 && fmt == 1) NSA_BW5_LAUNCH(128, 1)
  else if (a.D == 128) NSA_BW5_LAUNCH(128, 0)
  else if (fmt == 1) NSA_BW5_LAUNCH(64, 1)
  else NSA_BW5_LAUNCH(64, 0)
#undef NSA_BW5_LAUNCH
  return launch_status("selected backward (tcgen05)");
}

// Returns and clears the status word of the backward kernels (the stream has been synchronised by the caller).
int bw5_take_status(int* status) {
  int v = 0, zero = 0;
  NSA_CUDA_OK(cudaMemcpyFromSymbol(&v, g_bw5_status, sizeof(int)));
  if (v != 0) NSA_CUDA_OK(cudaMemcpyToSymbol(g_bw5_status, &zero, sizeof(int)));
  *status = v;
  return NSA_OK;
}

int bw5_set_status(int v) {
  NSA_CUDA_OK(cudaMemcpyToSymbol(g_bw5_status, &v, sizeof(int)));
  return NSA_OK;
}

}  // namespace nsa
