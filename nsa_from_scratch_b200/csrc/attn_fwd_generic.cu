// Generic NSA attention forward: every shape, block size, 16-bit type and the fp8 storage
// path.  One thread block owns a tile of TM = 16*NW query rows of one (batch, query head)
// and walks, branch by branch, the 64-key tiles that branch can see:
//   compressed : pooled tokens 0 .. hi(last row)            (Kc/Vc)
//   selected   : the listed blocks of the tile's query block (K/V rows blk*bn ..)
//   sliding    : the band lo(first row) .. hi(last row)      (K/V)
// Every branch reduces to "row i may attend keys lo_i <= j <= hi_i", so one masked
// streaming-softmax loop serves all three.  Tiles are staged with cp.async into a
// two-stage XOR-swizzled shared-memory ring; QK^T and PV run on mma.sync m16n8k16 with
// fp32 accumulation, P stays in registers.  In fused mode the gate-weighted sum of the
// branches is accumulated in shared memory and written once.
// This is the path for shapes the tcgen05 kernel does not take (D=32, blocks != 64,
// ragged lengths, fp8 storage); attn_fwd_tc5.cu is the performance path.
#include "common.cuh"

namespace nsa {

constexpr int TN = 64;         // keys per staged tile
constexpr int MAX_SEL = 256;   // listed blocks per query block this kernel can hold

struct FwdK {
  nsa_fwd_args a;
  int n_qtiles;      // query tiles per (b,h)
  int nk_blocks;     // selection KV blocks
  float scale_log2;  // softmax scale * log2(e)
};

// rows [row0, row0+TN) of a [*, D] 16-bit matrix -> swizzled smem tile; rows >= row_limit read as 0
template <typename T, int D, int NT>
__device__ __forceinline__ void stage_tile16(uint32_t sdst, const T* src, int row0, int nrows, int row_limit) {
  constexpr int CH = D / 8;
  for (int i = threadIdx.x; i < nrows * CH; i += NT) {
    int r = i / CH, c = i % CH;
    int gr = row0 + r;
    bool ok = gr < row_limit;
    const T* p = src + (size_t)(ok ? gr : 0) * D + c * 8;
    cp_async16(sdst + tile_off<D>(r, c), p, ok ? 16 : 0);
  }
}

// same for fp8 storage: dequantise to bf16(fp32(x) * scale) on the way in
template <int D, int NT>
__device__ __forceinline__ void stage_tile8(unsigned char* sdst, const uint8_t* src, int row0, int nrows,
                                            int row_limit, float scale, int fmt) {
  constexpr int CH = D / 8;
  for (int i = threadIdx.x; i < nrows * CH; i += NT) {
    int r = i / CH, c = i % CH;
    int gr = row0 + r;
    uint4 o = make_uint4(0, 0, 0, 0);
    if (gr < row_limit) {
      uint2 raw = *reinterpret_cast<const uint2*>(src + (size_t)gr * D + c * 8);
      const uint8_t* b = reinterpret_cast<const uint8_t*>(&raw);
      uint32_t w[4];
#pragma unroll
      for (int e = 0; e < 4; ++e)
        w[e] = Elem<__nv_bfloat16>::pack(fp8_to_f(b[2 * e], fmt) * scale, fp8_to_f(b[2 * e + 1], fmt) * scale);
      o = make_uint4(w[0], w[1], w[2], w[3]);
    }
    *reinterpret_cast<uint4*>(sdst + tile_off<D>(r, c)) = o;
  }
}

__device__ __forceinline__ float gate_logit(const void* g, size_t i, int dt) {
  if (dt == NSA_FP32) return reinterpret_cast<const float*>(g)[i];
  if (dt == NSA_FP16) return __half2float(reinterpret_cast<const __half*>(g)[i]);
  return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(g)[i]);
}

// Blocks per SM: at D <= 64 the register count is held to 128 so that four blocks are resident (the kernel is
// latency-bound: a selected-only launch with one list per head, B=2, T=32768, Hq=12, D=64, went 1.36 -> 0.99 ms).
template <typename T, int D, int NW, bool IN8>
__global__ void __launch_bounds__(NW * 32, D <= 64 ? 4 : 2) attn_fwd_generic_kernel(const __grid_constant__ FwdK p) {
  constexpr int TM = 16 * NW;
  constexpr int NT = 32 * NW;
  constexpr int CH = D / 8;
  constexpr int KS = D / 16;   // k-steps of QK^T == pairs of d-tiles of PV
  const nsa_fwd_args& a = p.a;

  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* Qs = smem;                               // TM x D, later the output staging tile
  unsigned char* KV = smem + TM * D * 2;                  // 2 stages x (K tile, V tile)
  // Fused launches: the gated sum of the finished branches, this thread's D/2 values.  Touched only at the two or
  // three branch ends, so it lives in local memory (volatile keeps it out of the registers, which the launch bound
  // holds to 128 at D <= 64, and out of shared memory, where its 16 KB per block cost a resident block per SM).
  volatile float total[2 * KS * 4];
  __shared__ int sel_list[MAX_SEL];
  __shared__ int sel_n;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int BH = a.B * a.H;
  const int qt = p.n_qtiles - 1 - (int)(blockIdx.x / BH);   // long rows first
  const int bh = (int)(blockIdx.x % BH);
  const int b = bh / a.H, h = bh % a.H;
  const int G = a.H / a.Hkv, hk = h / G;
  const int q0 = qt * TM;
  const int i_last = min(q0 + TM, a.Tq) - 1;

  const size_t q_slab = ((size_t)bh * a.Tq) * D;
  const size_t kv_slab = ((size_t)(b * a.Hkv + hk) * a.Tk) * D;
  const size_t kc_slab = ((size_t)(b * a.Hkv + hk) * a.Nc) * D;

  // ---- stage Q, build the list of selected blocks -------------------------------
  if constexpr (IN8) {
    stage_tile8<D, NT>(Qs, reinterpret_cast<const uint8_t*>(a.Q) + q_slab, q0, TM, a.Tq, a.q_scale, a.q_dtype);
  } else {
    stage_tile16<T, D, NT>(smem_u32(Qs), reinterpret_cast<const T*>(a.Q) + q_slab, q0, TM, a.Tq);
    cp_async_commit();
    cp_async_wait<0>();
  }
  if ((a.branches & NSA_BRANCH_SELECTED) && warp == 0) {
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

  uint32_t qf[KS][4];
#pragma unroll
  for (int ks = 0; ks < KS; ++ks)
    ldsm_x4(qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3],
            smem_u32(Qs) + tile_off<D>(warp * 16 + (lane & 15), ks * 2 + (lane >> 4)));

  const int g8 = lane >> 2, t4 = lane & 3;
  const int row_i[2] = {q0 + warp * 16 + g8, q0 + warp * 16 + g8 + 8};
  const bool row_ok[2] = {row_i[0] < a.Tq, row_i[1] < a.Tq};

  // gate values of the thread's two rows (fused mode)
  float gate[2][3] = {{0.5f, 0.5f, 0.5f}, {0.5f, 0.5f, 0.5f}};
  if (a.fused) {
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      float x[3] = {0.f, 0.f, 0.f};
      if (a.gates != nullptr && row_ok[r]) {
        size_t gi = ((a.io_layout & NSA_IO_GATES_BTHD) ? ((size_t)b * a.Tq + row_i[r]) * a.H + h
                                                       : (size_t)bh * a.Tq + row_i[r]) * 3;
#pragma unroll
        for (int c = 0; c < 3; ++c) x[c] = gate_logit(a.gates, gi + c, a.gate_dtype);
      }
      if (a.gate_act == NSA_GATE_SOFTMAX) {
        float mx = fmaxf(x[0], fmaxf(x[1], x[2]));
        float e0 = __expf(x[0] - mx), e1 = __expf(x[1] - mx), e2 = __expf(x[2] - mx);
        float inv = 1.f / (e0 + e1 + e2);
        gate[r][0] = e0 * inv; gate[r][1] = e1 * inv; gate[r][2] = e2 * inv;
      } else {
#pragma unroll
        for (int c = 0; c < 3; ++c) gate[r][c] = 1.f / (1.f + __expf(-x[c]));
      }
    }
  }

  float o[2 * KS][4];
  bool have_total = false;
  int last_branch = -1;
#pragma unroll
  for (int br = 0; br < 3; ++br) if (a.branches & (1 << br)) last_branch = br;

#pragma unroll 1
  for (int br = 0; br < 3; ++br) {
    if (!(a.branches & (1 << br))) continue;

    // ---- what this branch lets each row see -------------------------------------
    auto bounds = [&](int i, bool ok, int& lo, int& hi) {
      lo = 0; hi = -1;
      if (!ok) return;
      if (br == 0) {
        if (a.causal) {
          int num = i + a.cmp_offset - (a.cmp_block - 1);
          hi = num < 0 ? -1 : num / a.cmp_stride;
        } else hi = a.Nc - 1;
        hi = min(hi, a.Nc - 1);
      } else if (br == 1) {
        hi = a.causal ? min(i + a.offset, a.sel_key_limit - 1) : a.sel_key_limit - 1;
      } else {
        int pos = i + a.offset;
        if (a.causal) { lo = pos - a.window + 1; hi = pos; }
        else { lo = pos - a.window; hi = pos + a.window; }
        lo = max(lo, 0); hi = min(hi, a.Tk - 1);
      }
    };
    int lo[2], hi[2];
    bounds(row_i[0], row_ok[0], lo[0], hi[0]);
    bounds(row_i[1], row_ok[1], lo[1], hi[1]);

    int ntiles = 0, tile0 = 0, tpb = 1;
    {
      int lo_f, hi_f, lo_l, hi_l;
      bounds(q0, true, lo_f, hi_f);
      bounds(i_last, true, lo_l, hi_l);
      if (br == 0) ntiles = hi_l < 0 ? 0 : hi_l / TN + 1;
      else if (br == 1) { tpb = (a.bn + TN - 1) / TN; ntiles = sel_n * tpb; }
      else if (hi_l >= lo_f) { tile0 = lo_f / TN; ntiles = hi_l / TN - tile0 + 1; }
    }
    auto tile_start = [&](int t, int& j0, int& jlim) {
      if (br == 1) {
        int blk = sel_list[t / tpb];
        j0 = blk * a.bn + (t % tpb) * TN;
        jlim = min(blk * a.bn + a.bn, a.sel_key_limit);
      } else {
        j0 = (tile0 + t) * TN;
        jlim = br == 0 ? a.Nc : a.Tk;
      }
    };
    auto issue = [&](int t) {
      int j0, jlim;
      tile_start(t, j0, jlim);
      unsigned char* ks_ = KV + (t & 1) * (2 * TN * D * 2);
      unsigned char* vs_ = ks_ + TN * D * 2;
      if (br == 0) {
        stage_tile16<T, D, NT>(smem_u32(ks_), reinterpret_cast<const T*>(a.Kc) + kc_slab, j0, TN, a.Nc);
        stage_tile16<T, D, NT>(smem_u32(vs_), reinterpret_cast<const T*>(a.Vc) + kc_slab, j0, TN, a.Nc);
      } else if constexpr (IN8) {
        stage_tile8<D, NT>(ks_, reinterpret_cast<const uint8_t*>(a.K) + kv_slab, j0, TN, a.Tk, a.k_scale, a.kv_dtype);
        stage_tile8<D, NT>(vs_, reinterpret_cast<const uint8_t*>(a.V) + kv_slab, j0, TN, a.Tk, a.v_scale, a.kv_dtype);
      } else {
        stage_tile16<T, D, NT>(smem_u32(ks_), reinterpret_cast<const T*>(a.K) + kv_slab, j0, TN, a.Tk);
        stage_tile16<T, D, NT>(smem_u32(vs_), reinterpret_cast<const T*>(a.V) + kv_slab, j0, TN, a.Tk);
      }
      cp_async_commit();
    };

    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
#pragma unroll
    for (int d = 0; d < 2 * KS; ++d) { o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f; }

    if (ntiles > 0) issue(0);
#pragma unroll 1
    for (int t = 0; t < ntiles; ++t) {
      if (t + 1 < ntiles) { issue(t + 1); cp_async_wait<1>(); }
      else cp_async_wait<0>();
      __syncthreads();

      int j0, jlim;
      tile_start(t, j0, jlim);
      const uint32_t ks_ = smem_u32(KV + (t & 1) * (2 * TN * D * 2));
      const uint32_t vs_ = ks_ + TN * D * 2;

      // S = Q K^T
      float s[8][4];
#pragma unroll
      for (int n = 0; n < 8; ++n) { s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f; }
      const int mi = lane >> 3, r8 = lane & 7;
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
        for (int np = 0; np < 4; ++np) {
          uint32_t b0, b1, b2, b3;
          ldsm_x4(b0, b1, b2, b3, ks_ + tile_off<D>(np * 16 + (mi >> 1) * 8 + r8, ks * 2 + (mi & 1)));
          mma16816<T>(s[2 * np], qf[ks], b0, b1);
          mma16816<T>(s[2 * np + 1], qf[ks], b2, b3);
        }
      }

      // scale, mask, running softmax
      int hi_t[2] = {min(hi[0], jlim - 1), min(hi[1], jlim - 1)};
      bool full = lo[0] <= j0 && lo[1] <= j0 && hi_t[0] >= j0 + TN - 1 && hi_t[1] >= j0 + TN - 1;
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int n = 0; n < 8; ++n) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float v = s[n][e] * p.scale_log2;
          if (!full) {
            int j = j0 + n * 8 + t4 * 2 + (e & 1);
            int r = e >> 1;
            if (j < lo[r] || j > hi_t[r]) v = -INFINITY;
          }
          s[n][e] = v;
          mx[e >> 1] = fmaxf(mx[e >> 1], v);
        }
      }
      float alpha[2], msafe[2], ps[2] = {0.f, 0.f};
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        float mn = fmaxf(m[r], mx[r]);
        msafe[r] = mn == -INFINITY ? 0.f : mn;
        alpha[r] = ex2(m[r] - msafe[r]);     // m = -inf -> 0
        m[r] = mn;
      }
#pragma unroll
      for (int n = 0; n < 8; ++n) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float pv = ex2(s[n][e] - msafe[e >> 1]);
          s[n][e] = pv;
          ps[e >> 1] += pv;
        }
      }
#pragma unroll
      for (int r = 0; r < 2; ++r) l[r] = l[r] * alpha[r] + ps[r];
#pragma unroll
      for (int d = 0; d < 2 * KS; ++d) {
        o[d][0] *= alpha[0]; o[d][1] *= alpha[0]; o[d][2] *= alpha[1]; o[d][3] *= alpha[1];
      }

      // O += P V
#pragma unroll
      for (int kj = 0; kj < 4; ++kj) {
        uint32_t pa[4];
        pa[0] = Elem<T>::pack(s[2 * kj][0], s[2 * kj][1]);
        pa[1] = Elem<T>::pack(s[2 * kj][2], s[2 * kj][3]);
        pa[2] = Elem<T>::pack(s[2 * kj + 1][0], s[2 * kj + 1][1]);
        pa[3] = Elem<T>::pack(s[2 * kj + 1][2], s[2 * kj + 1][3]);
#pragma unroll
        for (int dp = 0; dp < KS; ++dp) {
          uint32_t b0, b1, b2, b3;
          ldsm_x4_t(b0, b1, b2, b3, vs_ + tile_off<D>(kj * 16 + (mi & 1) * 8 + r8, dp * 2 + (mi >> 1)));
          mma16816<T>(o[2 * dp], pa, b0, b1);
          mma16816<T>(o[2 * dp + 1], pa, b2, b3);
        }
      }
      __syncthreads();   // the stage is refilled by the next iteration's prefetch
    }

    // ---- finish the branch ---------------------------------------------------------
    float inv[2], lse_[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
      l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
      bool ok = l[r] > 0.f;
      inv[r] = ok ? 1.f / l[r] : 0.f;
      lse_[r] = ok ? m[r] * kLn2 + __logf(l[r]) : -INFINITY;
    }
    if (!a.fused) {
      if (a.lse != nullptr && t4 == 0) {
#pragma unroll
        for (int r = 0; r < 2; ++r)
          if (row_ok[r]) a.lse[(size_t)bh * a.Tq + row_i[r]] = lse_[r];
      }
#pragma unroll
      for (int d = 0; d < 2 * KS; ++d) {
        o[d][0] *= inv[0]; o[d][1] *= inv[0]; o[d][2] *= inv[1]; o[d][3] *= inv[1];
      }
    } else {
      float c0 = inv[0] * gate[0][br], c1 = inv[1] * gate[1][br];
      const bool last = br == last_branch;
#pragma unroll
      for (int d = 0; d < 2 * KS; ++d) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float v = o[d][e] * (e < 2 ? c0 : c1);
          if (have_total) v += total[d * 4 + e];
          if (last) o[d][e] = v; else total[d * 4 + e] = v;
        }
      }
      have_total = true;
    }
  }

  // ---- write the tile: registers -> staging tile -> 16-byte global stores ---------------
  __syncthreads();
#pragma unroll
  for (int d = 0; d < 2 * KS; ++d) {
    int col = d * 8 + t4 * 2;                 // element column; chunk = d, offset 4*t4 bytes
    uint32_t v0 = Elem<T>::pack(o[d][0], o[d][1]);
    uint32_t v1 = Elem<T>::pack(o[d][2], o[d][3]);
    int r0 = warp * 16 + g8;
    *reinterpret_cast<uint32_t*>(Qs + tile_off<D>(r0, d) + (col & 7) * 2) = v0;
    *reinterpret_cast<uint32_t*>(Qs + tile_off<D>(r0 + 8, d) + (col & 7) * 2) = v1;
  }
  __syncthreads();
  const bool bthd = (a.io_layout & NSA_IO_OUT_BTHD) != 0;           // rows H*D apart instead of D
  T* outp = reinterpret_cast<T*>(a.out) + (bthd ? ((size_t)b * a.Tq * a.H + h) * D : q_slab);
  const size_t row_stride = bthd ? (size_t)a.H * D : (size_t)D;
  for (int i = tid; i < TM * CH; i += NT) {
    int r = i / CH, c = i % CH;
    if (q0 + r < a.Tq)
      *reinterpret_cast<uint4*>(outp + (size_t)(q0 + r) * row_stride + c * 8) =
          *reinterpret_cast<const uint4*>(Qs + tile_off<D>(r, c));
  }
}

template <typename T, int D, int NW, bool IN8>
static int launch_generic(const FwdK& k, cudaStream_t st) {
  constexpr int TM = 16 * NW;
  size_t smem = (size_t)TM * D * 2 + 4 * (size_t)TN * D * 2;
  auto fn = attn_fwd_generic_kernel<T, D, NW, IN8>;
  NSA_CUDA_OK(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  long long blocks = (long long)k.a.B * k.a.H * k.n_qtiles;
  NSA_REQUIRE(blocks > 0 && blocks < 2147483647LL, NSA_ERR_ARG, "attention forward: %lld tiles do not fit a grid", blocks);
  fn<<<(unsigned)blocks, NW * 32, smem, st>>>(k);
  return launch_status("attn_fwd_generic");
}

template <typename T, bool IN8>
static int dispatch_d(const FwdK& k, int nw, cudaStream_t st) {
  switch (k.a.D) {
    case 32: return nw == 4 ? launch_generic<T, 32, 4, IN8>(k, st) : launch_generic<T, 32, 2, IN8>(k, st);
    case 64: return nw == 4 ? launch_generic<T, 64, 4, IN8>(k, st) : launch_generic<T, 64, 2, IN8>(k, st);
    case 128: return nw == 4 ? launch_generic<T, 128, 4, IN8>(k, st) : launch_generic<T, 128, 2, IN8>(k, st);
  }
  return fail(NSA_ERR_UNSUPPORTED, "attention forward: head dim %d not in {32,64,128}", k.a.D);
}

// Validated arguments -> launch.  Called by nsa_attention_fwd (abi.cu).
int attention_fwd_generic(const nsa_fwd_args& a, cudaStream_t st) {
  FwdK k;
  k.a = a;
  k.scale_log2 = a.scale * kLog2e;
  k.nk_blocks = a.bn > 0 ? (a.sel_key_limit + a.bn - 1) / a.bn : 0;
  int tm = 64;
  if (a.branches & NSA_BRANCH_SELECTED) {
    NSA_REQUIRE(a.top_k <= MAX_SEL, NSA_ERR_UNSUPPORTED, "selected: top_k %d > %d", a.top_k, MAX_SEL);
    if (a.bm % 64 != 0) {
      NSA_REQUIRE(a.bm == 32, NSA_ERR_UNSUPPORTED, "selected: block_size_m %d must be 32 or a multiple of 64", a.bm);
      tm = 32;
    }
  }
  k.n_qtiles = (a.Tq + tm - 1) / tm;
  const bool in8 = a.q_dtype == NSA_FP8_E4M3 || a.q_dtype == NSA_FP8_E5M2;
  if (in8) return dispatch_d<__nv_bfloat16, true>(k, tm / 16, st);
  if (a.q_dtype == NSA_FP16) return dispatch_d<__half, false>(k, tm / 16, st);
  return dispatch_d<__nv_bfloat16, false>(k, tm / 16, st);
}

}  // namespace nsa
