// Selection scores from the compressed branch's attention probabilities.
//
// score[b, hi, qb, j] = sum over the query block's rows i (and, for lists shared by a GQA group, over the
// group's query heads) of  sum_c p[i,c] * w(c,j),   p[i,c] = exp(q_i . Kc_c * scale - lse_i)  -- the
// probabilities of the compressed branch, recomputed from its log-sum-exp -- and w(c,j) the share of
// compressed token c's window [c*stride, c*stride + block) that lies in selection block j.
// One thread block owns (batch, index head, query block of 64 rows); per head it walks the visible
// compressed tokens in tiles of 64: S = Q Kc^T on mma.sync m16n8k16, P in registers, column sums over the 64
// rows (registers -> warp shuffles -> one slot per warp in shared memory, added in warp order), then every
// selection block gathers its up-to-(bn+block)/stride tokens with their weights.  No atomics: the sums are
// formed in a fixed order, so the scores (and the indices chosen from them) repeat bit for bit.
#include "common.cuh"

namespace nsa {

struct CmpScoreK {
  const void* Q;        // [B,H,Tq,D]
  const void* Kc;       // [B,Hkv,Nc,D]
  const float* lse;     // [B,H,Tq] natural-log lse of the compressed branch
  float* scores;        // [B,Hi,nq,nk]
  int B, H, Hkv, Hi, Tq, Nc, nq, nk;
  int cblock, cstride, cmp_offset, bn, sel_offset, causal, force_first, force_local;
  float scale_log2;
};

template <typename T, int D>
__global__ void __launch_bounds__(128, 2) cmp_scores_kernel(const CmpScoreK p) {
  constexpr int TM = 64, TN = 64, NT = 128, KS = D / 16, CH = D / 8;
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* Qs = smem;
  unsigned char* Ks = Qs + TM * D * 2;            // two buffers
  float* wsum = reinterpret_cast<float*>(Ks + 2 * TN * D * 2);   // [4][TN]
  float* csum = wsum + 4 * TN;                    // [2 * TN]: column sums of the previous and the current tile
  float* sc = csum + 2 * TN;                      // [nk]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g8 = lane >> 2, t4 = lane & 3, mi = lane >> 3, r8 = lane & 7;
  const int qb = blockIdx.x;
  const int bh = blockIdx.y, b = bh / p.Hi, hi = bh % p.Hi;
  const int G = p.H / p.Hkv;
  const int GS = p.Hi == p.H ? 1 : G;
  const int h0 = p.Hi == p.H ? hi : hi * G;
  const int hk = p.Hi == p.H ? hi / G : hi;
  const int q0 = qb * TM;
  const T* Kg = reinterpret_cast<const T*>(p.Kc) + ((size_t)(b * p.Hkv + hk) * p.Nc) * D;

  for (int j = tid; j < p.nk; j += NT) sc[j] = 0.f;

  // last compressed token a row may see
  auto hi_of = [&](int i) {
    if (!p.causal) return p.Nc - 1;
    const int num = i + p.cmp_offset - (p.cblock - 1);
    return min(num < 0 ? -1 : num / p.cstride, p.Nc - 1);
  };
  const int i_last = min(q0 + TM, p.Tq) - 1;
  const int n_vis = hi_of(i_last) + 1;            // tokens any row of the block sees
  const int ntiles = (n_vis + TN - 1) / TN;
  const int row_i[2] = {q0 + warp * 16 + g8, q0 + warp * 16 + g8 + 8};
  const int hi_r[2] = {row_i[0] < p.Tq ? hi_of(row_i[0]) : -1, row_i[1] < p.Tq ? hi_of(row_i[1]) : -1};

  auto stage_k = [&](int t, int buf) {
    const uint32_t dst = smem_u32(Ks + buf * TN * D * 2);
    for (int i = tid; i < TN * CH; i += NT) {
      const int r = i / CH, c = i % CH, gr = t * TN + r;
      const bool ok = gr < p.Nc;
      cp_async16(dst + tile_off<D>(r, c), Kg + (size_t)(ok ? gr : 0) * D + c * 8, ok ? 16 : 0);
    }
    cp_async_commit();
  };

#pragma unroll 1
  for (int gs = 0; gs < GS; ++gs) {
    const int h = h0 + gs;
    const size_t q_slab = ((size_t)(b * p.H + h) * p.Tq) * D;
    __syncthreads();                              // the previous head is done with Qs / Ks
    for (int i = tid; i < TM * CH; i += NT) {
      const int r = i / CH, c = i % CH, gr = q0 + r;
      const bool ok = gr < p.Tq;
      cp_async16(smem_u32(Qs) + tile_off<D>(r, c), reinterpret_cast<const T*>(p.Q) + q_slab + (size_t)(ok ? gr : 0) * D + c * 8, ok ? 16 : 0);
    }
    cp_async_commit();
    float lse2[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const float l = row_i[r] < p.Tq ? p.lse[(size_t)(b * p.H + h) * p.Tq + row_i[r]] : -INFINITY;
      lse2[r] = l * kLog2e;
    }
    if (ntiles > 0) stage_k(0, 0);
    for (int j = tid; j < 2 * TN; j += NT) csum[j] = 0.f;

#pragma unroll 1
    for (int t = 0; t < ntiles; ++t) {
      cp_async_wait<0>();
      __syncthreads();                            // tile t (and Q) landed; everyone is done with tile t-1's buffers
      if (t + 1 < ntiles) stage_k(t + 1, (t + 1) & 1);
      const uint32_t qs_ = smem_u32(Qs), ks_ = smem_u32(Ks + (t & 1) * TN * D * 2);
      float s[8][4];
#pragma unroll
      for (int n = 0; n < 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
        uint32_t qa[4];
        ldsm_x4(qa[0], qa[1], qa[2], qa[3], qs_ + tile_off<D>(warp * 16 + (lane & 15), ks * 2 + (lane >> 4)));
#pragma unroll
        for (int np = 0; np < 4; ++np) {
          uint32_t b0, b1, b2, b3;
          ldsm_x4(b0, b1, b2, b3, ks_ + tile_off<D>(np * 16 + (mi >> 1) * 8 + r8, ks * 2 + (mi & 1)));
          mma16816<T>(s[2 * np], qa, b0, b1);
          mma16816<T>(s[2 * np + 1], qa, b2, b3);
        }
      }
      // probabilities, summed over the warp's 16 rows per column
      const int c0 = t * TN;
#pragma unroll
      for (int n = 0; n < 8; ++n) {
        float cs[2];
#pragma unroll
        for (int e2 = 0; e2 < 2; ++e2) {
          const int c = c0 + n * 8 + t4 * 2 + e2;
          const float pa = (c <= hi_r[0] && lse2[0] > -INFINITY) ? ex2(fmaf(s[n][e2], p.scale_log2, -lse2[0])) : 0.f;
          const float pb = (c <= hi_r[1] && lse2[1] > -INFINITY) ? ex2(fmaf(s[n][2 + e2], p.scale_log2, -lse2[1])) : 0.f;
          float v = pa + pb;
          v += __shfl_xor_sync(0xffffffffu, v, 4);
          v += __shfl_xor_sync(0xffffffffu, v, 8);
          v += __shfl_xor_sync(0xffffffffu, v, 16);
          cs[e2] = v;
        }
        if (g8 == 0) { wsum[warp * TN + n * 8 + t4 * 2] = cs[0]; wsum[warp * TN + n * 8 + t4 * 2 + 1] = cs[1]; }
      }
      __syncthreads();
      // csum: [0,TN) = column sums of tile t-1, [TN,2TN) = of tile t (the four warps added in warp order)
      if (tid < TN) {
        csum[tid] = csum[TN + tid];
        csum[TN + tid] = ((wsum[tid] + wsum[TN + tid]) + wsum[2 * TN + tid]) + wsum[3 * TN + tid];
      }
      __syncthreads();
      // every selection block whose last visible token lies in this tile gathers its tokens, in token order; a block
      // spans at most (bn + block)/stride + 1 <= TN tokens (checked on the host), so they are all in the window
      const int tok_lo = t * TN, tok_hi = tok_lo + TN - 1, base = tok_lo - TN;
      // only blocks touched by this tile's tokens can end in it
      const int j_lo = (tok_lo * p.cstride) / p.bn;
      const int j_hi = min(p.nk - 1, (min(tok_hi, p.Nc - 1) * p.cstride + p.cblock - 1) / p.bn);
      for (int j = j_lo + tid; j <= j_hi; j += NT) {
        const int c_last = min(min(((j + 1) * p.bn - 1) / p.cstride, p.Nc - 1), n_vis - 1);   // last token starting inside the block
        const int num = j * p.bn - p.cblock + p.cstride;
        const int c_first = num < 0 ? 0 : num / p.cstride;                                     // first token whose window reaches it
        if (c_last < tok_lo || c_last > tok_hi || c_first > c_last) continue;
        float acc = 0.f;
        for (int c = c_first; c <= c_last; ++c) {
          const int w0 = max(c * p.cstride, j * p.bn), w1 = min(c * p.cstride + p.cblock, (j + 1) * p.bn);
          if (w1 <= w0) continue;
          acc = fmaf(csum[c - base], (float)(w1 - w0) / (float)p.cblock, acc);
        }
        sc[j] += acc;
      }
    }
  }
  __syncthreads();
  // legality and forced blocks, then out
  int cmax = p.nk - 1;
  if (p.causal) {
    const long long last = (long long)qb * TM + (TM - 1) + p.sel_offset;
    cmax = last < 0 ? -1 : (int)min((long long)(p.nk - 1), last / p.bn);
  }
  float* dst = p.scores + ((size_t)bh * p.nq + qb) * p.nk;
  for (int j = tid; j < p.nk; j += NT) {
    float v = sc[j];
    if (j > cmax) v = -INFINITY;
    else if (j < p.force_first || j > cmax - p.force_local) v = INFINITY;
    dst[j] = v;
  }
}

int cmp_block_scores(const void* Q, const void* Kc, const float* lse, float* scores, int B, int H, int Hkv, int Tq, int Nc, int D,
                     int nk, int cblock, int cstride, int cmp_offset, int bn, int sel_offset, int causal, float scale,
                     int force_first, int force_local, int shared, int dtype, cudaStream_t st) {
  NSA_REQUIRE(B > 0 && H > 0 && Hkv > 0 && H % Hkv == 0, NSA_ERR_ARG, "compressed scores: heads %d/%d", H, Hkv);
  NSA_REQUIRE(Tq > 0 && Nc > 0 && nk > 0, NSA_ERR_ARG, "compressed scores: empty problem");
  NSA_REQUIRE(cblock > 0 && cstride > 0 && cstride <= cblock && bn > 0, NSA_ERR_ARG, "compressed scores: block sizes");
  NSA_REQUIRE((bn + cblock) / cstride + 1 <= 64, NSA_ERR_UNSUPPORTED,
              "compressed scores: a selection block of %d keys spans more than 64 compressed tokens (block %d, stride %d)", bn, cblock, cstride);
  CmpScoreK k;
  k.Q = Q; k.Kc = Kc; k.lse = lse; k.scores = scores;
  k.B = B; k.H = H; k.Hkv = Hkv; k.Hi = shared ? Hkv : H; k.Tq = Tq; k.Nc = Nc; k.nq = (Tq + 63) / 64; k.nk = nk;
  k.cblock = cblock; k.cstride = cstride; k.cmp_offset = cmp_offset; k.bn = bn; k.sel_offset = sel_offset; k.causal = causal;
  k.force_first = force_first; k.force_local = force_local;
  k.scale_log2 = scale * kLog2e;
  NSA_REQUIRE((long long)B * k.Hi <= 65535, NSA_ERR_ARG, "compressed scores: B*H too large");
  dim3 grid((unsigned)k.nq, (unsigned)(B * k.Hi));
  const size_t smem = (size_t)64 * D * 2 * 3 + (4 * 64 + 2 * 64 + (size_t)nk) * 4;
  NSA_REQUIRE(smem <= 200 * 1024, NSA_ERR_UNSUPPORTED, "compressed scores: %d selection blocks exceed shared memory", nk);
#define NSA_CS(TT, DD)                                                                                   \
  {                                                                                                      \
    auto fn = cmp_scores_kernel<TT, DD>;                                                                 \
    NSA_CUDA_OK(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));      \
    fn<<<grid, 128, smem, st>>>(k);                                                                     \
  }
  if (dtype == NSA_BF16) {
    if (D == 128) NSA_CS(__nv_bfloat16, 128) else if (D == 64) NSA_CS(__nv_bfloat16, 64) else if (D == 32) NSA_CS(__nv_bfloat16, 32)
    else return fail(NSA_ERR_UNSUPPORTED, "compressed scores: head dim %d not in {32,64,128}", D);
  } else if (dtype == NSA_FP16) {
    if (D == 128) NSA_CS(__half, 128) else if (D == 64) NSA_CS(__half, 64) else if (D == 32) NSA_CS(__half, 32)
    else return fail(NSA_ERR_UNSUPPORTED, "compressed scores: head dim %d not in {32,64,128}", D);
  } else return fail(NSA_ERR_UNSUPPORTED, "compressed scores: dtype %d", dtype);
#undef NSA_CS
  return launch_status("cmp_block_scores");
}

}  // namespace nsa
