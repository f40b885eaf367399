// Selection scores from the compressed branch's attention probabilities on the 5th-generation tensor cores.
//
// Same definition as cmp_scores.cu (the mma.sync kernel, which stays for the shapes this one does not take):
//   hs[b,h,qb,j] = sum over the 64 rows i of query block qb of  sum_c exp(q_i . Kc_c * scale - lse_i) * w(c,j).
// The product is formed TRANSPOSED: S^T = Kc_tile . Q_X^T, so a TMEM lane is a compressed token and its
// 128 columns are the query rows of tile X.  The sum over query rows -- the reduction the scorer needs -- is then a
// sum over one thread's registers: no shuffles, no P written back, no second MMA.  The probabilities need no
// running maximum (the log-sum-exp is an input), so S^T is double-buffered in TMEM and the tensor pipe runs a
// tile ahead of the exponentials.
//
// Work item as in the attention kernel: 4 row groups (query head, query block) that share one KV head = two
// 128-row tiles X.  Warp 0: TMA producer (Q once, pooled-K tiles of 128 tokens into a ring).  Warp 1: MMA issuer.
// Warps 4-7 / 8-11: tile 0 / tile 1 -- exponentials and row-group sums per token, left in a two-tile window of
// token sums in shared memory.  Warps 2 / 3: for tile 0 / 1, every selection block whose last token lies in the
// newest tile gathers its tokens (overlap weights) from the window, off the critical path.  All sums are formed
// in a fixed order.  Every wait is bounded; a wait that gives up raises the block's abort flag and the device
// status word, and the block still frees its TMEM.
#include "common.cuh"
#include "tc5_ptx.cuh"

#include <cudaTypedefs.h>

namespace nsa {

using namespace tc5;

int make_map(CUtensorMap* m, const void* ptr, long long slabs, long long rows, int D, int dtype);   // attn_fwd_tc5.cu

__device__ int g_cs5_status;

struct Cs5Params {
  CUtensorMap tmQ, tmKc;
  const float* lse;     // [B,H,Tq]
  float* hs;            // [B,H,nq,nk] per-head block sums (no legality, no forcing)
  int B, H, Hkv, Tq, Nc, nq, nk;
  int cblock, cstride, cmp_offset, bn, causal;
  float scale_log2;
  int GH, HG, NQG, NST;
  int tpb, wpt;         // token starts per selection block (bn / stride), strides per compression window (block / stride)
};

enum { C_QFULL = 0, C_KFULL = 1, C_KEMPTY = 5, C_SFULL = 9, C_SFREE = 13, C_TOK = 17, C_GAT = 19, C_COUNT = 21 };
// K*: up to 4 stages; S*: 2*X + buffer; TOK (per tile X, 128 arrivals): token sums written; GAT (1 arrival): blocks gathered

template <int D, int FMT>
__global__ void __launch_bounds__(384, 1) cmp_scores_tc5_kernel(const __grid_constant__ Cs5Params p) {
  constexpr int DH = D / 64;
  constexpr int QTILE = DH * 128 * 128;
  constexpr int KTILE = DH * 128 * 128;
  constexpr int DHSTRIDE = 128 * 128;
  constexpr int TT = 128;                          // tokens per tile

  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sQ = smem_u32(smem);
  const uint32_t sK = sQ + 2 * QTILE;
  float* lse2s = reinterpret_cast<float*>(smem + 2 * QTILE + p.NST * KTILE);   // [256] -lse*log2(e) per row of the item (-inf: row sees nothing)
  float* tokv = lse2s + 256;                                                    // [2 tiles][2 X][2 groups][128 tokens]
  float* sc = tokv + 2 * 2 * 2 * TT;                                            // [4 groups][nk]
  __shared__ __align__(8) uint64_t bars[C_COUNT];
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_flag;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int per_q = p.B * p.Hkv * p.HG;
  const int qbg = p.NQG - 1 - (int)(blockIdx.x / per_q);
  const int rem = (int)(blockIdx.x % per_q);
  const int b = rem / (p.Hkv * p.HG);
  const int hk = (rem / p.HG) % p.Hkv;
  const int hg = rem % p.HG;
  const int G = p.H / p.Hkv;
  const int GH = p.GH, NQB = 4 / p.GH;
  const int h_base = hk * G + hg * GH;
  const int qb_base = qbg * NQB;
  auto grp_head = [&](int g) { return h_base + g % GH; };
  auto grp_qb = [&](int g) { return qb_base + g / GH; };
  auto bar = [&](int id) { return smem_u32(&bars[id]); };

  // last compressed token row i may see
  auto hi_of = [&](int i) {
    if (!p.causal) return p.Nc - 1;
    const int num = i + p.cmp_offset - (p.cblock - 1);
    return min(num < 0 ? -1 : num / p.cstride, p.Nc - 1);
  };
  const int i_last = min(min(qb_base + NQB, p.nq) * 64, p.Tq) - 1;
  const int n_vis = hi_of(i_last) + 1;
  const int ntiles = (n_vis + TT - 1) / TT;

  if (tid == 0) {
    abort_flag = 0;
    for (int i = 0; i < C_COUNT; ++i) mbar_init(bar(i), (i >= C_SFREE && i < C_GAT) ? 128 : 1);
    fence_barrier_init();
  }
  if (warp == 1) { tmem_alloc(smem_u32(&tmem_base_s), 512); tmem_relinquish(); }
  // rows of the item: r = 64*g + position; -lse*log2(e), or -inf for rows that do not exist or see nothing
  for (int r = tid; r < 256; r += blockDim.x) {
    const int g = r >> 6, qi = grp_qb(g) * 64 + (r & 63);
    float v = -INFINITY;
    if (grp_qb(g) < p.nq && qi < p.Tq) {
      const float l = p.lse[((size_t)b * p.H + grp_head(g)) * p.Tq + qi];
      if (l > -INFINITY) v = -l * kLog2e;
    }
    lse2s[r] = v;
  }
  for (int i = tid; i < 2 * 2 * 2 * TT + 4 * p.nk; i += blockDim.x) tokv[i] = 0.f;   // tokv and sc are contiguous
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_s;
  int fail_id = 0;
  int last_k_t = -1;

  if (warp == 0) {
    // =============================== TMA producer ===============================
    const bool leader = elect_one();
    if (leader) {
      tma_prefetch_desc(&p.tmQ); tma_prefetch_desc(&p.tmKc);
      mbar_expect_tx(bar(C_QFULL), 2 * QTILE);
      for (int X = 0; X < 2; ++X)
        for (int hh = 0; hh < 2; ++hh)
          for (int dh = 0; dh < DH; ++dh)
            tma_load_3d(sQ + X * QTILE + dh * DHSTRIDE + hh * 8192, &p.tmQ, bar(C_QFULL), dh * 64, grp_qb(2 * X + hh) * 64,
                        b * p.H + grp_head(2 * X + hh));
    }
    __syncwarp();
    bool ok = true;
    for (int t = 0; t < ntiles && ok; ++t) {
      const int s = t % p.NST, ph = (t / p.NST) & 1;
      ok = __all_sync(0xffffffffu, mbar_wait(bar(C_KEMPTY + s), ph ^ 1, &abort_flag));
      if (!ok) { fail_id = C_KEMPTY + s + 1; break; }
      if (leader) {
        mbar_expect_tx(bar(C_KFULL + s), KTILE);
        for (int c = 0; c < 2; ++c)
          for (int dh = 0; dh < DH; ++dh)
            tma_load_3d(sK + s * KTILE + dh * DHSTRIDE + c * 8192, &p.tmKc, bar(C_KFULL + s), dh * 64, t * TT + c * 64, b * p.Hkv + hk);
      }
      last_k_t = t;
      __syncwarp();
    }
  } else if (warp == 1) {
    // =============================== MMA issuer: S^T_X = Kc_tile . Q_X^T ===============================
    const bool leader = elect_one();
    constexpr uint32_t IDESC = idesc_f16(FMT, 128, 128, 0, 0);
    bool ok = __all_sync(0xffffffffu, mbar_wait(bar(C_QFULL), 0, &abort_flag));
    if (!ok) fail_id = C_QFULL + 1;
    const uint64_t dQ[2] = {smem_desc_sw128(sQ, 16, 1024), smem_desc_sw128(sQ + QTILE, 16, 1024)};
    for (int t = 0; t < ntiles && ok; ++t) {
      const int s = t % p.NST, ph = (t / p.NST) & 1;
      ok = __all_sync(0xffffffffu, mbar_wait(bar(C_KFULL + s), ph, &abort_flag));
      if (!ok) { fail_id = C_KFULL + s + 1; break; }
      tc_fence_after();
      const uint64_t dK = smem_desc_sw128(sK + s * KTILE, 16, 1024);
#pragma unroll
      for (int X = 0; X < 2; ++X) {
        if (!ok) break;
        // buffer t&1 of tile X is free once its previous contents (tile t-2) have been read
        ok = __all_sync(0xffffffffu, mbar_wait(bar(C_SFREE + 2 * X + (t & 1)), ((t >> 1) & 1) ^ 1, &abort_flag));
        if (!ok) { fail_id = C_SFREE + 2 * X + (t & 1) + 1; break; }
        tc_fence_after();
        if (leader) {
          const uint32_t tS = tmem + (uint32_t)((2 * X + (t & 1)) * 128);
#pragma unroll
          for (int ks = 0; ks < D / 16; ++ks) {
            const uint32_t off = (uint32_t)(((ks >> 2) * DHSTRIDE + (ks & 3) * 32) >> 4);
            if (ks == 0) mma_ss(tS, dK + off, dQ[X] + off, IDESC, 0u);
            else mma_ss(tS, dK + off, dQ[X] + off, IDESC, 1u);
          }
          tc_commit(bar(C_SFULL + 2 * X + (t & 1)));
          if (X == 1) tc_commit(bar(C_KEMPTY + s));
        }
        __syncwarp();
      }
    }
  } else if (warp >= 4) {
    // =============================== exponentials, token sums, block gather ===============================
    const int X = (warp - 4) >> 2;
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;                       // token of the tile == TMEM lane
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const float sl2 = p.scale_log2;
    // the two row groups of this tile
    int g_qb[2], g_rows[2];
#pragma unroll
    for (int gg = 0; gg < 2; ++gg) {
      g_qb[gg] = grp_qb(2 * X + gg);
      g_rows[gg] = g_qb[gg] < p.nq ? min(64, p.Tq - g_qb[gg] * 64) : 0;        // rows of the group that exist
    }
    const int last_tok = ntiles * TT - 1;
    bool ok = true;
#pragma unroll 1
    for (int t = 0; t < ntiles && ok; ++t) {
      const int bsel = t & 1;
      ok = __all_sync(0xffffffffu, mbar_wait(bar(C_SFULL + 2 * X + bsel), (t >> 1) & 1, &abort_flag));
      if (!ok) { fail_id = C_SFULL + 2 * X + bsel + 1; break; }
      tc_fence_after();
      uint32_t sv[4][32];
      const uint32_t tS = tmem + lane_addr + (uint32_t)((2 * X + bsel) * 128);
      tmem_ld32(tS, sv[0]);
      tmem_ld32(tS + 32, sv[1]);
      tmem_ld32(tS + 64, sv[2]);
      tmem_ld32(tS + 96, sv[3]);
      tc_wait_ld();
      tc_fence_before();
      mbar_arrive(bar(C_SFREE + 2 * X + bsel));              // S^T is in registers: the MMA warp may refill the buffer
      const int c = t * TT + r;                              // this thread's compressed token
      float tsum[2];
#pragma unroll
      for (int gg = 0; gg < 2; ++gg) {
        // rows of the group that see token c: positions >= c*stride + block - 1 - cmp_offset (causal), and existing
        int vlo = 0;
        if (p.causal) vlo = max(0, c * p.cstride + p.cblock - 1 - p.cmp_offset - g_qb[gg] * 64);
        const int vhi = c < p.Nc ? g_rows[gg] : 0;           // exclusive
        const float4* ls4 = reinterpret_cast<const float4*>(lse2s + (2 * X + gg) * 64);
        float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
        if (vlo == 0 && vhi == 64) {
#pragma unroll
          for (int q = 0; q < 2; ++q)
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
              const float4 l4 = ls4[q * 8 + (i >> 2)];
              s0 += ex2(fmaf(__uint_as_float(sv[2 * gg + q][i]), sl2, l4.x));
              s1 += ex2(fmaf(__uint_as_float(sv[2 * gg + q][i + 1]), sl2, l4.y));
              s2 += ex2(fmaf(__uint_as_float(sv[2 * gg + q][i + 2]), sl2, l4.z));
              s3 += ex2(fmaf(__uint_as_float(sv[2 * gg + q][i + 3]), sl2, l4.w));
            }
        } else if (vlo < vhi) {
#pragma unroll
          for (int q = 0; q < 2; ++q)
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
              const float4 l4 = ls4[q * 8 + (i >> 2)];
              const float lv[4] = {l4.x, l4.y, l4.z, l4.w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const int col = q * 32 + i + e;
                const float pv = (col >= vlo && col < vhi) ? ex2(fmaf(__uint_as_float(sv[2 * gg + q][i + e]), sl2, lv[e])) : 0.f;
                if (e == 0) s0 += pv; else if (e == 1) s1 += pv; else if (e == 2) s2 += pv; else s3 += pv;
              }
            }
        }
        tsum[gg] = (s0 + s1) + (s2 + s3);
      }
      // slot t&1 held tile t-2, which the gather of tile t-1 still reads; that gather started when this tile's
      // exponentials did, so the wait is over long before it is reached.  (It also keeps the TOK barrier at most one
      // phase ahead of the gather warp, which waits on its phases by parity.)
      if (t >= 1) {
        ok = __all_sync(0xffffffffu, mbar_wait(bar(C_GAT + X), (t - 1) & 1, &abort_flag));
        if (!ok) { fail_id = C_GAT + X + 1; break; }
      }
      tokv[(((t & 1) * 2 + X) * 2 + 0) * TT + r] = tsum[0];
      tokv[(((t & 1) * 2 + X) * 2 + 1) * TT + r] = tsum[1];
      mbar_arrive(bar(C_TOK + X));                           // 128 arrivals: the tile's token sums are in the ring
    }
  } else {
    // =============================== block gather (warp 2: tile 0, warp 3: tile 1) ===============================
    // Selection blocks whose last token lies in tile t gather their tokens from ring slots t and t-1 (a block spans
    // at most 64 tokens); lanes take (row group, block) tasks; sc is only ever touched by this warp.
    const int X = warp - 2;
    const int last_tok = ntiles * TT - 1;
    bool ok = true;
#pragma unroll 1
    for (int t = 0; t < ntiles && ok; ++t) {
      ok = __all_sync(0xffffffffu, mbar_wait(bar(C_TOK + X), t & 1, &abort_flag));
      if (!ok) { fail_id = C_TOK + X + 1; break; }
      // In units of the stride: a selection block holds tpb token starts, a window spans wpt of them; token
      // c = j*tpb + u (u from -(wpt-1) to tpb-1) overlaps block j by min(u + wpt, tpb) - max(u, 0) units of its wpt.
      // Block j is gathered in the tile that holds its last token start (clipped to the last token processed).
      const int tok_lo = t * TT, tok_hi = min(tok_lo + TT - 1, last_tok);
      const int tpb = p.tpb, wpt = p.wpt;
      const int j_lo = tok_lo / tpb;                                           // first block whose last token start is in the tile
      const int j_top = t == ntiles - 1 ? min(p.nk - 1, (tok_hi + wpt - 1) / tpb)   // last tile: every block a processed token reaches
                                        : (tok_lo + TT - tpb) / tpb;
      const float inv_wpt = 1.f / (float)wpt;
      for (int gg = 0; gg < 2; ++gg) {
        for (int j = j_lo + lane; j <= j_top; j += 32) {
          const int c_end = min(j * tpb + tpb - 1, tok_hi);                   // last token start of the block that was processed
          if (c_end < tok_lo) continue;
          float acc = 0.f;
          for (int u = -(wpt - 1); u < tpb; ++u) {
            const int cc = j * tpb + u;
            if (cc < 0 || cc > c_end) continue;
            const int ov = min(u + wpt, tpb) - max(u, 0);
            const int tt = cc >> 7;                                            // t or t-1
            acc = fmaf(tokv[((((tt & 1) * 2 + X) * 2 + gg) * TT) + (cc & (TT - 1))], (float)ov * inv_wpt, acc);
          }
          sc[(2 * X + gg) * p.nk + j] += acc;
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(C_GAT + X));            // the slot of tile t-1 may be overwritten
    }
  }

  if (fail_id != 0) atomicCAS(&g_cs5_status, 0, fail_id);
  tc_fence_before();
  __syncthreads();
  if (abort_flag && warp == 0 && lane == 0) {
    for (int i = 0; i < 20000 && !mbar_try_wait(bar(C_QFULL), 0); ++i) __nanosleep(100);
    if (last_k_t >= 0)
      for (int i = 0; i < 20000 && !mbar_try_wait(bar(C_KFULL + last_k_t % p.NST), (last_k_t / p.NST) & 1); ++i) __nanosleep(100);
  }
  // per-head block sums out (rows of groups that exist)
  if (!abort_flag) {
    for (int g = 0; g < 4; ++g) {
      if (grp_qb(g) >= p.nq) continue;
      float* dst = p.hs + (((size_t)b * p.H + grp_head(g)) * p.nq + grp_qb(g)) * p.nk;
      for (int j = tid; j < p.nk; j += blockDim.x) dst[j] = sc[g * p.nk + j];
    }
  }
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, 512); }
}

// scores[b,hi,qb,j] = (sum over the index head's query heads, in head order, of) hs, -inf where the block is
// causally illegal for the query block, +inf where it is forced
__global__ void __launch_bounds__(256) cmp_scores_finish_kernel(const float* __restrict__ hs, float* __restrict__ scores, int H,
                                                                int Hi, int nq, int nk, int bn, int sel_offset, int causal,
                                                                int force_first, int force_local, long long total) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int j = (int)(i % nk);
    const long long row = i / nk;
    const int qb = (int)(row % nq);
    const long long bhi = row / nq;
    const int hi = (int)(bhi % Hi);
    const long long b = bhi / Hi;
    const int GS = H / Hi;
    float v = hs[((b * H + (long long)hi * GS) * nq + qb) * nk + j];
    for (int gs = 1; gs < GS; ++gs) v = __fadd_rn(v, hs[((b * H + (long long)hi * GS + gs) * nq + qb) * nk + j]);
    int cmax = nk - 1;
    if (causal) {
      const long long last = (long long)qb * 64 + 63 + sel_offset;
      cmax = last < 0 ? -1 : (int)min((long long)(nk - 1), last / bn);
    }
    if (j > cmax) v = -INFINITY;
    else if (j < force_first || j > cmax - force_local) v = INFINITY;
    scores[i] = v;
  }
}

bool cmp_scores_tc5_supports(int D, int dtype, int cblock, int cstride, int bn, int nk) {
  if (!(D == 64 || D == 128)) return false;
  if (!(dtype == NSA_BF16 || dtype == NSA_FP16)) return false;
  if ((bn + cblock) / cstride + 1 > 64) return false;
  if (bn % cstride != 0 || cblock % cstride != 0) return false;      // the gather works in units of the stride
  // Q tiles + 2 K stages + row data + token window + 4 score rows must fit
  const size_t need = (size_t)4 * (D / 64) * 128 * 128 + (256 + 8 * 128 + (size_t)4 * nk) * 4 + 1024;
  return need <= 225 * 1024;
}

int cmp_block_scores_tc5(const void* Q, const void* Kc, const float* lse, float* scores, float* head_scratch, int B, int H, int Hkv,
                         int Tq, int Nc, int D, int nk, int cblock, int cstride, int cmp_offset, int bn, int sel_offset,
                         int causal, float scale, int force_first, int force_local, int shared, int dtype, cudaStream_t st) {
  Cs5Params p;
  int rc;
  if ((rc = make_map(&p.tmQ, Q, (long long)B * H, Tq, D, dtype)) != NSA_OK) return rc;
  if ((rc = make_map(&p.tmKc, Kc, (long long)B * Hkv, Nc, D, dtype)) != NSA_OK) return rc;
  p.lse = lse; p.hs = head_scratch;
  p.B = B; p.H = H; p.Hkv = Hkv; p.Tq = Tq; p.Nc = Nc; p.nq = (Tq + 63) / 64; p.nk = nk;
  p.cblock = cblock; p.cstride = cstride; p.cmp_offset = cmp_offset; p.bn = bn; p.causal = causal;
  p.scale_log2 = scale * kLog2e;
  p.tpb = bn / cstride; p.wpt = cblock / cstride;
  const int G = H / Hkv;
  p.GH = G % 4 == 0 ? 4 : (G % 2 == 0 ? 2 : 1);
  p.HG = G / p.GH;
  p.NQG = (p.nq + 4 / p.GH - 1) / (4 / p.GH);
  const size_t tile = (size_t)(D / 64) * 128 * 128;
  const size_t fixed = 2 * tile + (256 + 8 * 128 + (size_t)4 * nk) * 4 + 1024;
  int nst = (int)((225 * 1024 - fixed) / tile);
  p.NST = nst > 4 ? 4 : nst;
  NSA_REQUIRE(p.NST >= 2, NSA_ERR_UNSUPPORTED, "compressed scores: %d selection blocks leave no room for the key ring", nk);
  const size_t smem = fixed + p.NST * tile;
  const long long blocks = (long long)p.NQG * B * Hkv * p.HG;
  NSA_REQUIRE(blocks > 0 && blocks < 2147483647LL, NSA_ERR_ARG, "compressed scores: %lld work items do not fit a grid", blocks);
#define NSA_CS5(DD, FF)                                                                                  \
  {                                                                                                      \
    auto fn = cmp_scores_tc5_kernel<DD, FF>;                                                             \
    NSA_CUDA_OK(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));      \
    fn<<<(unsigned)blocks, 384, smem, st>>>(p);                                                         \
  }
  const int fmt = dtype == NSA_BF16 ? 1 : 0;
  if (D == 128 && fmt == 1) NSA_CS5(128, 1) else if (D == 128) NSA_CS5(128, 0) else if (fmt == 1) NSA_CS5(64, 1) else NSA_CS5(64, 0)
#undef NSA_CS5
  rc = launch_status("cmp_scores_tc5");
  if (rc != NSA_OK) return rc;
  const int Hi = shared ? Hkv : H;
  const long long total = (long long)B * Hi * p.nq * nk;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const long long want = (total + 255) / 256;
  const int grid = (int)(want < (long long)sms * 16 ? (want < 1 ? 1 : want) : (long long)sms * 16);
  cmp_scores_finish_kernel<<<grid, 256, 0, st>>>(head_scratch, scores, H, Hi, p.nq, nk, bn, sel_offset, causal, force_first, force_local, total);
  return launch_status("cmp_scores_finish");
}

int cs5_take_status(int* status) {
  int v = 0, zero = 0;
  NSA_CUDA_OK(cudaMemcpyFromSymbol(&v, g_cs5_status, sizeof(int)));
  if (v != 0) NSA_CUDA_OK(cudaMemcpyToSymbol(g_cs5_status, &zero, sizeof(int)));
  *status = v;
  return NSA_OK;
}

}  // namespace nsa
