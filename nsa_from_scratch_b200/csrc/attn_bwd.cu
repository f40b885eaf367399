// Attention backward for one NSA branch per launch: selected (the KV blocks listed for the query
// block), sliding (the band of keys the tile's rows can see) or compressed (the pooled tokens; K/V are
// then the pooled tensors and dK/dV their gradients, which nsa_pool_mean_bwd spreads back over the
// rows).  One thread block owns a tile of TM = 16*NW query rows of one (batch, query head).  Per 64-key tile:
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

// Blocks per SM: the kernel is latency-bound (mma.sync chains, atomics), so at D <= 64 the register count is held
// to 128 for four resident blocks (2.86 -> 2.68 ms at B=2, T=32768, Hq=12, Hkv=1, D=64); at D=128 shared memory
// (80 KB per block) allows two.
template <typename T, int D, int NW>
__global__ void __launch_bounds__(NW * 32, (D <= 64 ? 16 : 8) / NW) selected_bwd_kernel(const __grid_constant__ BwdK p) {
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
  const int key_rows = a.branch == NSA_BRANCH_COMPRESSED ? a.Nc : a.Tk;   // rows of K/V (and of dK/dV)
  const size_t kv_slab = ((size_t)(b * a.Hkv + hk) * key_rows) * D;
  const T* Kg = reinterpret_cast<const T*>(a.K) + kv_slab;
  const T* Vg = reinterpret_cast<const T*>(a.V) + kv_slab;

  bstage16<T, D, NT>(smem_u32(Qs), reinterpret_cast<const T*>(a.Q) + q_slab, q0, TM, a.Tq);
  bstage16<T, D, NT>(smem_u32(dOs), reinterpret_cast<const T*>(a.dO) + q_slab, q0, TM, a.Tq);
  cp_async_commit();
  // what the branch lets a query row see: keys lo..hi (inclusive)
  auto bounds = [&](int i, int& lo, int& hi) {
    lo = 0;
    if (a.branch == NSA_BRANCH_COMPRESSED) {
      if (a.causal) {
        const int num = i + a.cmp_offset - (a.cmp_block - 1);
        hi = num < 0 ? -1 : num / a.cmp_stride;
      } else hi = a.Nc - 1;
      hi = min(hi, a.Nc - 1);
    } else if (a.branch == NSA_BRANCH_SLIDING) {
      const int pos = i + a.offset;
      if (a.causal) { lo = pos - a.window + 1; hi = pos; }
      else { lo = pos - a.window; hi = pos + a.window; }
      lo = max(lo, 0); hi = min(hi, a.Tk - 1);
    } else {
      hi = a.causal ? min(i + a.offset, a.sel_key_limit - 1) : a.sel_key_limit - 1;
    }
  };
  if (warp == 0) {
    int n = 0;
    if (a.branch == NSA_BRANCH_SELECTED) {
      const int qb = q0 / a.bm;
      const int hi_ = (a.Hi == a.H) ? h : hk;
      const int32_t* row = a.idx + (((size_t)b * a.Hi + hi_) * a.nq + qb) * a.top_k;
      const int last_pos = i_last + a.offset;
      for (int s0 = 0; s0 < a.top_k; s0 += 32) {
        int s = s0 + lane;
        int blk = s < a.top_k ? row[s] : -1;
        bool ok = blk >= 0 && blk < p.nk_blocks && (!a.causal || (long long)blk * a.bn <= last_pos);
        unsigned m = __ballot_sync(0xffffffffu, ok);
        if (ok) sel_list[n + __popc(m & ((1u << lane) - 1))] = blk;
        n += __popc(m);
      }
    }
    if (lane == 0) sel_n = n;
  }
  __syncthreads();
  const int tpb = (a.bn + BTN - 1) / BTN;
  int ntiles = 0, tile0 = 0;
  if (a.branch == NSA_BRANCH_SELECTED) ntiles = sel_n * tpb;
  else {
    int lo_f, hi_f, lo_l, hi_l;
    bounds(q0, lo_f, hi_f);
    bounds(i_last, lo_l, hi_l);
    if (a.branch == NSA_BRANCH_COMPRESSED) ntiles = hi_l < 0 ? 0 : hi_l / BTN + 1;
    else if (hi_l >= lo_f) { tile0 = lo_f / BTN; ntiles = hi_l / BTN - tile0 + 1; }
  }

  const int g8 = lane >> 2, t4 = lane & 3, mi = lane >> 3, r8 = lane & 7;
  const int row_l[2] = {warp * 16 + g8, warp * 16 + g8 + 8};
  const int row_i[2] = {q0 + row_l[0], q0 + row_l[1]};
  float lse2[2], dl[2];
  int lo[2], hi[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    bool ok = row_i[r] < a.Tq;
    float l = ok ? a.lse[(size_t)bh * a.Tq + row_i[r]] : -INFINITY;
    dl[r] = ok ? a.delta[(size_t)bh * a.Tq + row_i[r]] : 0.f;
    ok = ok && l > -INFINITY;
    lse2[r] = ok ? l * kLog2e : 0.f;
    bounds(row_i[r], lo[r], hi[r]);
    if (!ok) hi[r] = -1;
  }

  float dq[2 * KS][4];
#pragma unroll
  for (int d = 0; d < 2 * KS; ++d) { dq[d][0] = dq[d][1] = dq[d][2] = dq[d][3] = 0.f; }

  auto tile_start = [&](int t, int& j0, int& jlim) {
    if (a.branch == NSA_BRANCH_SELECTED) {
      int blk = sel_list[t / tpb];
      j0 = blk * a.bn + (t % tpb) * BTN;
      jlim = min(blk * a.bn + a.bn, a.sel_key_limit);
    } else {
      j0 = (tile0 + t) * BTN;
      jlim = key_rows;
    }
  };
  auto issue = [&](int t) {
    int j0, jlim;
    tile_start(t, j0, jlim);
    bstage16<T, D, NT>(smem_u32(Ks), Kg, j0, BTN, key_rows);
    bstage16<T, D, NT>(smem_u32(Vs), Vg, j0, BTN, key_rows);
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
        float pv = (j >= lo[r] && j <= hi_t[r]) ? ex2(s[n][e] * p.scale_log2 - lse2[r]) : 0.f;
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
    // Four warps cover the tile's 64 keys, 16 each.  With eight warps (128 query rows) warps 0-3 form dV while warps
    // 4-7 form dK; with fewer, every warp does both in turn.
    constexpr int NPASS = NW >= 8 ? 1 : 2;
#pragma unroll 1
    for (int pi = 0; pi < NPASS; ++pi) {
      const int pass = NW >= 8 ? (warp >> 2) : pi;
      const uint32_t as_ = smem_u32(pass == 0 ? Ps : dSs);
      const uint32_t bs_ = pass == 0 ? dos_ : qs_;
      float* dst = pass == 0 ? dVg : dKg;
#pragma unroll 1
      for (int mt = (NW >= 8 ? (warp & 3) : warp); mt < 4; mt += (NW >= 8 ? 4 : NW)) {
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
        const int key_lim = min(jlim, key_rows);
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
    case 64: return nw == 8 ? launch_bwd<T, 64, 8>(k, st) : nw == 4 ? launch_bwd<T, 64, 4>(k, st) : launch_bwd<T, 64, 2>(k, st);
    case 128: return nw == 4 ? launch_bwd<T, 128, 4>(k, st) : launch_bwd<T, 128, 2>(k, st);
  }
  return fail(NSA_ERR_UNSUPPORTED, "selected backward: head dim %d not in {32,64,128}", k.a.D);
}

int attention_bwd(const nsa_bwd_args& a, cudaStream_t st) {
  BwdK k;
  k.a = a;
  k.scale_log2 = a.scale * kLog2e;
  k.nk_blocks = 0;
  int tm = 64;
  if (a.branch == NSA_BRANCH_SELECTED) {
    k.nk_blocks = (a.sel_key_limit + a.bn - 1) / a.bn;
    NSA_REQUIRE(a.top_k <= BMAX_SEL, NSA_ERR_UNSUPPORTED, "selected backward: top_k %d > %d", a.top_k, BMAX_SEL);
    if (a.bm % 64 != 0) {
      NSA_REQUIRE(a.bm == 32, NSA_ERR_UNSUPPORTED, "selected backward: block_size_m %d must be 32 or a multiple of 64", a.bm);
      tm = 32;
    }
  }
  // Compressed and sliding branches at D=64: 128 query rows per block, so that a K/V tile is fetched, and its dK/dV
  // partial sums are added atomically, once per 128 rows instead of once per 64.
  else if (a.D == 64 && a.Tq >= 128) tm = 128;
  k.n_qtiles = (a.Tq + tm - 1) / tm;
  if (a.dtype == NSA_BF16) return bwd_dispatch<__nv_bfloat16>(k, tm / 16, st);
  if (a.dtype == NSA_FP16) return bwd_dispatch<__half>(k, tm / 16, st);
  return fail(NSA_ERR_UNSUPPORTED, "selected backward: dtype %d", a.dtype);
}

// ------------------------------------------------------------------ pooling backward
// dX[j] += sum over the windows c that cover row j of dXc[c] / block  (fp32 in, fp32 accumulate into dX).
__global__ void __launch_bounds__(256) pool_mean_bwd_kernel(const float* __restrict__ dxc, float* __restrict__ dx, int Tlen,
                                                            int D, int block, int stride, int n_out) {
  const int CH = D / 4;
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)Tlen * CH) return;
  const int j = (int)(i / CH), ch = (int)(i % CH);
  // windows c with c*stride <= j <= c*stride + block - 1
  int c_hi = j / stride;
  int c_lo = j - (block - 1) <= 0 ? 0 : (j - (block - 1) + stride - 1) / stride;
  c_hi = min(c_hi, n_out - 1);
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  const float4* src = reinterpret_cast<const float4*>(dxc + (size_t)blockIdx.y * n_out * D) + ch;
  for (int c = c_lo; c <= c_hi; ++c) {
    const float4 v = src[(size_t)c * CH];
    acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
  }
  const float inv = 1.f / (float)block;
  float4* dst = reinterpret_cast<float4*>(dx + (size_t)blockIdx.y * Tlen * D) + (size_t)j * CH + ch;
  float4 o = *dst;
  o.x += acc.x * inv; o.y += acc.y * inv; o.z += acc.z * inv; o.w += acc.w * inv;
  *dst = o;
}

int pool_mean_bwd(const float* dxc, float* dx, int B, int H, int T, int D, int block, int stride, int n_out, cudaStream_t st) {
  NSA_REQUIRE(D % 4 == 0 && D > 0, NSA_ERR_ARG, "pool backward: D %d must be a positive multiple of 4", D);
  NSA_REQUIRE(block > 0 && stride > 0 && stride <= block, NSA_ERR_ARG, "pool backward: block %d stride %d", block, stride);
  if (n_out == 0 || T == 0 || B * H == 0) return NSA_OK;
  NSA_REQUIRE((long long)B * H <= 65535, NSA_ERR_ARG, "pool backward: B*H too large");
  dim3 grid((unsigned)(((long long)T * (D / 4) + 255) / 256), (unsigned)(B * H));
  pool_mean_bwd_kernel<<<grid, 256, 0, st>>>(dxc, dx, T, D, block, stride, n_out);
  return launch_status("pool_mean_bwd");
}

}  // namespace nsa
