// Selected-branch backward.  One thread block owns a tile of TM = 16*NW query rows of one
// (batch, query head) and walks the KV blocks listed for its query block.  Per 64-key tile:
//   S  = Q K^T            P  = exp(S*scale - lse)        (masked entries 0)
//   dP = dO V^T           dS = P * (dP - delta) * scale
//   dQ += dS K                                   (registers, written once at the end)
//   dV += P^T dO          dK += dS^T Q           (fp32 atomic adds into [B,Hkv,Tk,D])
// All five products run on mma.sync m16n8k16 with fp32 accumulation; P and dS are staged
// in shared memory as 16-bit so that their transposes can be read back with ldmatrix.trans.
// The next tile's K/V are fetched with cp.async while dV/dK are being formed.
#include "common.cuh"

namespace nsa {

constexpr int BTN = 64;
constexpr int BMAX_SEL = 256;

struct BwdK {
  nsa_bwd_args a;
  int n_qtiles;
  int nk_blocks;
  float scale_log2;
};

template <typename T, int D, int NT>
__device__ __forceinline__ void bstage16(uint32_t sdst, const T* src, int row0, int nrows, int row_limit) {
  constexpr int CH = D / 8;
  for (int i = threadIdx.x; i < nrows * CH; i += NT) {
    int r = i / CH, c = i % CH;
    int gr = row0 + r;
    bool ok = gr < row_limit;
    cp_async16(sdst + tile_off<D>(r, c), src + (size_t)(ok ? gr : 0) * D + c * 8, ok ? 16 : 0);
  }
}

template <typename T, int D, int NW>
__global__ void __launch_bounds__(NW * 32, 2) selected_bwd_kernel(const __grid_constant__ BwdK p) {
  constexpr int TM = 16 * NW;
  constexpr int NT = 32 * NW;
  constexpr int KS = D / 16;
  const nsa_bwd_args& a = p.a;

  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* Qs = smem;
  unsigned char* dOs = Qs + TM * D * 2;
  unsigned char* Ks = dOs + TM * D * 2;
  unsigned char* Vs = Ks + BTN * D * 2;
  unsigned char* Ps = Vs + BTN * D * 2;        // [TM][64]
  unsigned char* dSs = Ps + TM * BTN * 2;      // [TM][64]
  __shared__ int sel_list[BMAX_SEL];
  __shared__ int sel_n;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int BH = a.B * a.H;
  const int qt = (int)(blockIdx.x / BH);
  const int bh = (int)(blockIdx.x % BH);
  const int b = bh / a.H, h = bh % a.H;
  const int hk = h / (a.H / a.Hkv);
  const int q0 = qt * TM;
  const int i_last = min(q0 + TM, a.Tq) - 1;
  const size_t q_slab = ((size_t)bh * a.Tq) * D;
  const size_t kv_slab = ((size_t)(b * a.Hkv + hk) * a.Tk) * D;
  const T* Kg = reinterpret_cast<const T*>(a.K) + kv_slab;
  const T* Vg = reinterpret_cast<const T*>(a.V) + kv_slab;

  bstage16<T, D, NT>(smem_u32(Qs), reinterpret_cast<const T*>(a.Q) + q_slab, q0, TM, a.Tq);
  bstage16<T, D, NT>(smem_u32(dOs), reinterpret_cast<const T*>(a.dO) + q_slab, q0, TM, a.Tq);
  cp_async_commit();
  if (warp == 0) {
    const int qb = q0 / a.bm;
    const int hi_ = (a.Hi == a.H) ? h : hk;
    const int32_t* row = a.idx + (((size_t)b * a.Hi + hi_) * a.nq + qb) * a.top_k;
    const int last_pos = i_last + a.offset;
    int n = 0;
    for (int s0 = 0; s0 < a.top_k; s0 += 32) {
      int s = s0 + lane;
      int blk = s < a.top_k ? row[s] : -1;
      bool ok = blk >= 0 && blk < p.nk_blocks && (!a.causal || (long long)blk * a.bn <= last_pos);
      unsigned m = __ballot_sync(0xffffffffu, ok);
      if (ok) sel_list[n + __popc(m & ((1u << lane) - 1))] = blk;
      n += __popc(m);
    }
    if (lane == 0) sel_n = n;
  }
  __syncthreads();
  const int tpb = (a.bn + BTN - 1) / BTN;
  const int ntiles = sel_n * tpb;

  const int g8 = lane >> 2, t4 = lane & 3, mi = lane >> 3, r8 = lane & 7;
  const int row_l[2] = {warp * 16 + g8, warp * 16 + g8 + 8};
  const int row_i[2] = {q0 + row_l[0], q0 + row_l[1]};
  float lse2[2], dl[2];
  int hi[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    bool ok = row_i[r] < a.Tq;
    float l = ok ? a.lse[(size_t)bh * a.Tq + row_i[r]] : -INFINITY;
    dl[r] = ok ? a.delta[(size_t)bh * a.Tq + row_i[r]] : 0.f;
    ok = ok && l > -INFINITY;
    lse2[r] = ok ? l * kLog2e : 0.f;
    hi[r] = !ok ? -1 : (a.causal ? min(row_i[r] + a.offset, a.sel_key_limit - 1) : a.sel_key_limit - 1);
  }

  float dq[2 * KS][4];
#pragma unroll
  for (int d = 0; d < 2 * KS; ++d) { dq[d][0] = dq[d][1] = dq[d][2] = dq[d][3] = 0.f; }

  auto tile_start = [&](int t, int& j0, int& jlim) {
    int blk = sel_list[t / tpb];
    j0 = blk * a.bn + (t % tpb) * BTN;
    jlim = min(blk * a.bn + a.bn, a.sel_key_limit);
  };
  auto issue = [&](int t) {
    int j0, jlim;
    tile_start(t, j0, jlim);
    bstage16<T, D, NT>(smem_u32(Ks), Kg, j0, BTN, a.Tk);
    bstage16<T, D, NT>(smem_u32(Vs), Vg, j0, BTN, a.Tk);
    cp_async_commit();
  };
  if (ntiles > 0) issue(0);

#pragma unroll 1
  for (int t = 0; t < ntiles; ++t) {
    cp_async_wait<0>();
    __syncthreads();
    int j0, jlim;
    tile_start(t, j0, jlim);
    const uint32_t qs_ = smem_u32(Qs), dos_ = smem_u32(dOs), ks_ = smem_u32(Ks), vs_ = smem_u32(Vs);

    float s[8][4], dp[8][4];
#pragma unroll
    for (int n = 0; n < 8; ++n) {
      s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
      dp[n][0] = dp[n][1] = dp[n][2] = dp[n][3] = 0.f;
    }
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      uint32_t qa[4], da[4];
      ldsm_x4(qa[0], qa[1], qa[2], qa[3], qs_ + tile_off<D>(warp * 16 + (lane & 15), ks * 2 + (lane >> 4)));
      ldsm_x4(da[0], da[1], da[2], da[3], dos_ + tile_off<D>(warp * 16 + (lane & 15), ks * 2 + (lane >> 4)));
#pragma unroll
      for (int np = 0; np < 4; ++np) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4(b0, b1, b2, b3, ks_ + tile_off<D>(np * 16 + (mi >> 1) * 8 + r8, ks * 2 + (mi & 1)));
        mma16816<T>(s[2 * np], qa, b0, b1);
        mma16816<T>(s[2 * np + 1], qa, b2, b3);
        ldsm_x4(b0, b1, b2, b3, vs_ + tile_off<D>(np * 16 + (mi >> 1) * 8 + r8, ks * 2 + (mi & 1)));
        mma16816<T>(dp[2 * np], da, b0, b1);
        mma16816<T>(dp[2 * np + 1], da, b2, b3);
      }
    }
    // P and dS in place (s <- P, dp <- dS), staged to shared memory as 16-bit
    const int hi_t[2] = {min(hi[0], jlim - 1), min(hi[1], jlim - 1)};
#pragma unroll
    for (int n = 0; n < 8; ++n) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int r = e >> 1;
        const int j = j0 + n * 8 + t4 * 2 + (e & 1);
        float pv = j <= hi_t[r] ? ex2(s[n][e] * p.scale_log2 - lse2[r]) : 0.f;
        s[n][e] = pv;
        dp[n][e] = pv * (dp[n][e] - dl[r]) * a.scale;
      }
      const uint32_t off0 = tile_off<64>(row_l[0], n) + t4 * 4, off1 = tile_off<64>(row_l[1], n) + t4 * 4;
      *reinterpret_cast<uint32_t*>(Ps + off0) = Elem<T>::pack(s[n][0], s[n][1]);
      *reinterpret_cast<uint32_t*>(Ps + off1) = Elem<T>::pack(s[n][2], s[n][3]);
      *reinterpret_cast<uint32_t*>(dSs + off0) = Elem<T>::pack(dp[n][0], dp[n][1]);
      *reinterpret_cast<uint32_t*>(dSs + off1) = Elem<T>::pack(dp[n][2], dp[n][3]);
    }
    // dQ += dS K
#pragma unroll
    for (int kj = 0; kj < 4; ++kj) {
      uint32_t pa[4];
      pa[0] = Elem<T>::pack(dp[2 * kj][0], dp[2 * kj][1]);
      pa[1] = Elem<T>::pack(dp[2 * kj][2], dp[2 * kj][3]);
      pa[2] = Elem<T>::pack(dp[2 * kj + 1][0], dp[2 * kj + 1][1]);
      pa[3] = Elem<T>::pack(dp[2 * kj + 1][2], dp[2 * kj + 1][3]);
#pragma unroll
      for (int dd = 0; dd < KS; ++dd) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4_t(b0, b1, b2, b3, ks_ + tile_off<D>(kj * 16 + (mi & 1) * 8 + r8, dd * 2 + (mi >> 1)));
        mma16816<T>(dq[2 * dd], pa, b0, b1);
        mma16816<T>(dq[2 * dd + 1], pa, b2, b3);
      }
    }
    __syncthreads();                       // P/dS visible; K/V tiles free
    if (t + 1 < ntiles) issue(t + 1);

    // dV += P^T dO and dK += dS^T Q : 16 keys per pass
    float* dVg = a.dV_f + kv_slab;
    float* dKg = a.dK_f + kv_slab;
#pragma unroll 1
    for (int pass = 0; pass < 2; ++pass) {
      const uint32_t as_ = smem_u32(pass == 0 ? Ps : dSs);
      const uint32_t bs_ = pass == 0 ? dos_ : qs_;
      float* dst = pass == 0 ? dVg : dKg;
#pragma unroll 1
      for (int mt = warp; mt < 4; mt += NW) {
        float acc[2 * KS][4];
#pragma unroll
        for (int d = 0; d < 2 * KS; ++d) { acc[d][0] = acc[d][1] = acc[d][2] = acc[d][3] = 0.f; }
#pragma unroll
        for (int kq = 0; kq < NW; ++kq) {   // 16 query rows per step
          uint32_t ta[4];
          ldsm_x4_t(ta[0], ta[1], ta[2], ta[3], as_ + tile_off<64>(kq * 16 + (mi >> 1) * 8 + r8, mt * 2 + (mi & 1)));
#pragma unroll
          for (int dd = 0; dd < KS; ++dd) {
            uint32_t b0, b1, b2, b3;
            ldsm_x4_t(b0, b1, b2, b3, bs_ + tile_off<D>(kq * 16 + (mi & 1) * 8 + r8, dd * 2 + (mi >> 1)));
            mma16816<T>(acc[2 * dd], ta, b0, b1);
            mma16816<T>(acc[2 * dd + 1], ta, b2, b3);
          }
        }
        const int key0 = j0 + mt * 16 + g8, key1 = key0 + 8;
        const int key_lim = min(jlim, a.Tk);
#pragma unroll
        for (int d = 0; d < 2 * KS; ++d) {
          const int col = d * 8 + t4 * 2;
          if (key0 < key_lim) atomicAdd(reinterpret_cast<float2*>(dst + (size_t)key0 * D + col), make_float2(acc[d][0], acc[d][1]));
          if (key1 < key_lim) atomicAdd(reinterpret_cast<float2*>(dst + (size_t)key1 * D + col), make_float2(acc[d][2], acc[d][3]));
        }
      }
    }
  }

  // dQ
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    if (row_i[r] >= a.Tq) continue;
    const size_t base = q_slab + (size_t)row_i[r] * D;
#pragma unroll
    for (int d = 0; d < 2 * KS; ++d) {
      const int col = d * 8 + t4 * 2;
      float x = dq[d][2 * r], y = dq[d][2 * r + 1];
      if (a.dq_dtype == NSA_FP32) *reinterpret_cast<float2*>(reinterpret_cast<float*>(a.dQ) + base + col) = make_float2(x, y);
      else *reinterpret_cast<uint32_t*>(reinterpret_cast<T*>(a.dQ) + base + col) = Elem<T>::pack(x, y);
    }
  }
}

template <typename T, int D, int NW>
static int launch_bwd(const BwdK& k, cudaStream_t st) {
  constexpr int TM = 16 * NW;
  size_t smem = 2 * (size_t)TM * D * 2 + 2 * (size_t)BTN * D * 2 + 2 * (size_t)TM * BTN * 2;
  auto fn = selected_bwd_kernel<T, D, NW>;
  NSA_CUDA_OK(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  long long blocks = (long long)k.a.B * k.a.H * k.n_qtiles;
  NSA_REQUIRE(blocks > 0 && blocks < 2147483647LL, NSA_ERR_ARG, "selected backward: %lld tiles do not fit a grid", blocks);
  fn<<<(unsigned)blocks, NW * 32, smem, st>>>(k);
  return launch_status("selected_bwd");
}

template <typename T>
static int bwd_dispatch(const BwdK& k, int nw, cudaStream_t st) {
  switch (k.a.D) {
    case 32: return nw == 4 ? launch_bwd<T, 32, 4>(k, st) : launch_bwd<T, 32, 2>(k, st);
    case 64: return nw == 4 ? launch_bwd<T, 64, 4>(k, st) : launch_bwd<T, 64, 2>(k, st);
    case 128: return nw == 4 ? launch_bwd<T, 128, 4>(k, st) : launch_bwd<T, 128, 2>(k, st);
  }
  return fail(NSA_ERR_UNSUPPORTED, "selected backward: head dim %d not in {32,64,128}", k.a.D);
}

int selected_bwd(const nsa_bwd_args& a, cudaStream_t st) {
  BwdK k;
  k.a = a;
  k.scale_log2 = a.scale * kLog2e;
  k.nk_blocks = (a.sel_key_limit + a.bn - 1) / a.bn;
  NSA_REQUIRE(a.top_k <= BMAX_SEL, NSA_ERR_UNSUPPORTED, "selected backward: top_k %d > %d", a.top_k, BMAX_SEL);
  int tm = 64;
  if (a.bm % 64 != 0) {
    NSA_REQUIRE(a.bm == 32, NSA_ERR_UNSUPPORTED, "selected backward: block_size_m %d must be 32 or a multiple of 64", a.bm);
    tm = 32;
  }
  k.n_qtiles = (a.Tq + tm - 1) / tm;
  if (a.dtype == NSA_BF16) return bwd_dispatch<__nv_bfloat16>(k, tm / 16, st);
  if (a.dtype == NSA_FP16) return bwd_dispatch<__half>(k, tm / 16, st);
  return fail(NSA_ERR_UNSUPPORTED, "selected backward: dtype %d", a.dtype);
}

}  // namespace nsa
