// Block mean pooling, block scoring + top-k selection.  HBM/latency-bound integer-output
// work: coalesced 128-bit loads, fp32 arithmetic on CUDA cores in a fixed order (the
// selected indices must equal the reference's, so every rounding point is reproduced:
// fp32 sum of the block's rows, exact divide, one rounding to the 16-bit type, fp32 fma
// dot over D in index order, scale applied last).
#include "common.cuh"

namespace nsa {

// ------------------------------------------------------------------ pooling
// One thread produces 8 consecutive columns of one pooled row.
template <typename T, bool IN8>
__global__ void __launch_bounds__(256) pool_mean_kernel(const void* __restrict__ xin, T* __restrict__ out, int Tlen, int D,
                                                        int block, int stride, int n_out, float dq, int fmt) {
  const int CH = D / 8;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_out * CH) return;
  const int c = i / CH, ch = i % CH;
  const size_t slab = (size_t)blockIdx.y * Tlen * D;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  const int r0 = c * stride;
  const int r1 = min(r0 + block, Tlen);
  for (int r = r0; r < r1; ++r) {
    if constexpr (IN8) {
      const uint8_t* p = reinterpret_cast<const uint8_t*>(xin) + slab + (size_t)r * D + ch * 8;
      uint2 raw = *reinterpret_cast<const uint2*>(p);
      const uint8_t* b = reinterpret_cast<const uint8_t*>(&raw);
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] += Elem<T>::to_f(Elem<T>::from_f(fp8_to_f(b[e], fmt) * dq));
    } else {
      const T* p = reinterpret_cast<const T*>(xin) + slab + (size_t)r * D + ch * 8;
      uint4 raw = *reinterpret_cast<const uint4*>(p);
      const uint32_t* w = reinterpret_cast<const uint32_t*>(&raw);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float2 f = Elem<T>::unpack(w[e]);
        acc[2 * e] += f.x;
        acc[2 * e + 1] += f.y;
      }
    }
  }
  const float inv_n = (float)block;
  uint32_t w[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) w[e] = Elem<T>::pack(__fdiv_rn(acc[2 * e], inv_n), __fdiv_rn(acc[2 * e + 1], inv_n));
  T* q = out + ((size_t)blockIdx.y * n_out + c) * D + ch * 8;
  *reinterpret_cast<uint4*>(q) = make_uint4(w[0], w[1], w[2], w[3]);
}

// Learned pooling: out[c, d] = sum_s x[c*stride + s, d] * w[s, d] over the `block` rows of the window (rows past the
// end of the sequence count as zero), fp32 sum in row order, one rounding to the 16-bit type.
template <typename T>
__global__ void __launch_bounds__(256) pool_weighted_kernel(const T* __restrict__ x, const float* __restrict__ wgt, T* __restrict__ out,
                                                            int Tlen, int D, int block, int stride, int n_out) {
  const int CH = D / 8;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_out * CH) return;
  const int c = i / CH, ch = i % CH;
  const size_t slab = (size_t)blockIdx.y * Tlen * D;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  const int r0 = c * stride;
  const int r1 = min(r0 + block, Tlen);
  for (int r = r0; r < r1; ++r) {
    const uint4 raw = *reinterpret_cast<const uint4*>(x + slab + (size_t)r * D + ch * 8);
    const uint32_t* w = reinterpret_cast<const uint32_t*>(&raw);
    const float4 g0 = *reinterpret_cast<const float4*>(wgt + (size_t)(r - r0) * D + ch * 8);
    const float4 g1 = *reinterpret_cast<const float4*>(wgt + (size_t)(r - r0) * D + ch * 8 + 4);
    const float g[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = Elem<T>::unpack(w[e]);
      acc[2 * e] = fmaf(f.x, g[2 * e], acc[2 * e]);
      acc[2 * e + 1] = fmaf(f.y, g[2 * e + 1], acc[2 * e + 1]);
    }
  }
  uint32_t w[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) w[e] = Elem<T>::pack(acc[2 * e], acc[2 * e + 1]);
  *reinterpret_cast<uint4*>(out + ((size_t)blockIdx.y * n_out + c) * D + ch * 8) = make_uint4(w[0], w[1], w[2], w[3]);
}

int pool_weighted(const void* x, const float* w, void* out, int B, int H, int T, int D, int block, int stride, int n_out, int dtype,
                  cudaStream_t st) {
  NSA_REQUIRE(D % 8 == 0 && D > 0, NSA_ERR_ARG, "pool: D %d must be a positive multiple of 8", D);
  NSA_REQUIRE(block > 0 && stride > 0 && stride <= block, NSA_ERR_ARG, "pool: need 0 < stride <= block (%d, %d)", stride, block);
  const int expect = stride == block ? (T + block - 1) / block : (T >= block ? (T - block) / stride + 1 : 0);
  NSA_REQUIRE(n_out == expect, NSA_ERR_ARG, "pool: n_out %d, expected %d", n_out, expect);
  NSA_REQUIRE((reinterpret_cast<uintptr_t>(w) & 15) == 0, NSA_ERR_ARG, "pool: weights must be 16-byte aligned");
  if (n_out == 0 || B * H == 0) return NSA_OK;
  NSA_REQUIRE((long long)B * H <= 65535, NSA_ERR_ARG, "pool: B*H %lld too large", (long long)B * H);
  dim3 grid((unsigned)(((long long)n_out * (D / 8) + 255) / 256), (unsigned)(B * H));
  switch (dtype) {
    case NSA_BF16: pool_weighted_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, w, (__nv_bfloat16*)out, T, D, block, stride, n_out); break;
    case NSA_FP16: pool_weighted_kernel<__half><<<grid, 256, 0, st>>>((const __half*)x, w, (__half*)out, T, D, block, stride, n_out); break;
    default: return fail(NSA_ERR_UNSUPPORTED, "pool (learned): dtype %d", dtype);
  }
  return launch_status("pool_weighted");
}

int pool_mean(const void* x, void* out, int B, int H, int T, int D, int block, int stride, int n_out, int dtype,
              float dq, cudaStream_t st) {
  NSA_REQUIRE(D % 8 == 0 && D > 0, NSA_ERR_ARG, "pool: D %d must be a positive multiple of 8", D);
  NSA_REQUIRE(block > 0 && stride > 0 && stride <= block, NSA_ERR_ARG, "pool: need 0 < stride <= block (%d, %d)", stride, block);
  int expect = stride == block ? (T + block - 1) / block : (T >= block ? (T - block) / stride + 1 : 0);
  NSA_REQUIRE(n_out == expect, NSA_ERR_ARG, "pool: n_out %d, expected %d", n_out, expect);
  if (n_out == 0 || B * H == 0) return NSA_OK;
  NSA_REQUIRE((long long)B * H <= 65535, NSA_ERR_ARG, "pool: B*H %lld too large", (long long)B * H);
  dim3 grid((unsigned)(((long long)n_out * (D / 8) + 255) / 256), (unsigned)(B * H));
  switch (dtype) {
    case NSA_BF16: pool_mean_kernel<__nv_bfloat16, false><<<grid, 256, 0, st>>>(x, (__nv_bfloat16*)out, T, D, block, stride, n_out, 1.f, 0); break;
    case NSA_FP16: pool_mean_kernel<__half, false><<<grid, 256, 0, st>>>(x, (__half*)out, T, D, block, stride, n_out, 1.f, 0); break;
    case NSA_FP8_E4M3:
    case NSA_FP8_E5M2: pool_mean_kernel<__nv_bfloat16, true><<<grid, 256, 0, st>>>(x, (__nv_bfloat16*)out, T, D, block, stride, n_out, dq, dtype); break;
    default: return fail(NSA_ERR_UNSUPPORTED, "pool: dtype %d", dtype);
  }
  return launch_status("pool_mean");
}

// ------------------------------------------------------------------ KV-cache append
// One launch brings a cache up to date with t_new appended positions: the rows go into K and V, and the pooled
// windows and selection-block means that contain a new row are recomputed with pool_mean_kernel's arithmetic
// (fp32 sum in row order, divide by the window size, one rounding).  Rows at or past `filled` are read from
// the new tensors, so nothing in the launch depends on another thread's copy.
// One thread = 8 columns of one item; items of a slab: t_new row copies, nw pooled windows, nbk block means.
template <typename T>
__global__ void __launch_bounds__(256) cache_append_kernel(const T* __restrict__ k_new, const T* __restrict__ v_new,
                                                           T* __restrict__ K, T* __restrict__ V, T* __restrict__ Kc,
                                                           T* __restrict__ Vc, T* __restrict__ Kb, int D, int t_new,
                                                           int filled, int max_len, int nc_alloc, int nb_alloc, int cblock,
                                                           int cstride, int c0, int nw, int sblock, int b0, int nbk,
                                                           const int32_t* __restrict__ dyn_filled) {
  const int CH = D / 8;
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (dyn_filled != nullptr) {
    // fill count in device memory (a captured graph replays this launch as the cache grows): the window and block
    // ranges are derived here; the grid was sized for the largest they can be
    filled = *dyn_filled;
    const int T1d = filled + t_new;
    if (T1d > max_len) return;                             // the host refuses this before launching; never write past the end
    auto n_pooled = [&](int len) { return cstride == cblock ? (len + cblock - 1) / cblock : (len >= cblock ? (len - cblock) / cstride + 1 : 0); };
    c0 = cstride == cblock ? filled / cblock : n_pooled(filled);
    nw = min(n_pooled(T1d), nc_alloc) - c0;
    b0 = filled / sblock;
    nbk = min((T1d + sblock - 1) / sblock, nb_alloc) - b0;
  }
  const long long items = (long long)t_new + nw + nbk;
  if (i >= items * CH) return;
  const int item = (int)(i / CH), ch = (int)(i % CH);
  const size_t slab = blockIdx.y;
  const int T1 = filled + t_new;
  auto row8 = [&](const T* cache, const T* fresh, int r) {
    const T* p = r >= filled ? fresh + (slab * t_new + (r - filled)) * D : cache + (slab * max_len + r) * D;
    return *reinterpret_cast<const uint4*>(p + ch * 8);
  };
  auto mean8 = [&](const T* cache, const T* fresh, int r0, int block) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    const int r1 = min(r0 + block, T1);
    for (int rb = r0; rb < r1; rb += 8) {                  // eight rows' loads in flight, added in row order
      uint4 raw[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) raw[j] = rb + j < r1 ? row8(cache, fresh, rb + j) : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (rb + j < r1) {
          const uint32_t w[4] = {raw[j].x, raw[j].y, raw[j].z, raw[j].w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 f = Elem<T>::unpack(w[e]);
            acc[2 * e] += f.x;
            acc[2 * e + 1] += f.y;
          }
        }
      }
    }
    const float n = (float)block;
    return make_uint4(Elem<T>::pack(__fdiv_rn(acc[0], n), __fdiv_rn(acc[1], n)), Elem<T>::pack(__fdiv_rn(acc[2], n), __fdiv_rn(acc[3], n)),
                      Elem<T>::pack(__fdiv_rn(acc[4], n), __fdiv_rn(acc[5], n)), Elem<T>::pack(__fdiv_rn(acc[6], n), __fdiv_rn(acc[7], n)));
  };
  if (item < t_new) {
    const size_t dst = (slab * max_len + filled + item) * D + ch * 8, src = (slab * t_new + item) * D + ch * 8;
    *reinterpret_cast<uint4*>(K + dst) = *reinterpret_cast<const uint4*>(k_new + src);
    *reinterpret_cast<uint4*>(V + dst) = *reinterpret_cast<const uint4*>(v_new + src);
  } else if (item < t_new + nw) {
    const int c = c0 + (item - t_new);
    const size_t dst = (slab * nc_alloc + c) * D + ch * 8;
    *reinterpret_cast<uint4*>(Kc + dst) = mean8(K, k_new, c * cstride, cblock);
    *reinterpret_cast<uint4*>(Vc + dst) = mean8(V, v_new, c * cstride, cblock);
  } else {
    const int bb = b0 + (item - t_new - nw);
    *reinterpret_cast<uint4*>(Kb + (slab * nb_alloc + bb) * D + ch * 8) = mean8(K, k_new, bb * sblock, sblock);
  }
}

__global__ void cache_advance_kernel(int32_t* filled, int t_new, int max_len) {
  if (threadIdx.x == 0 && blockIdx.x == 0 && *filled + t_new <= max_len) *filled += t_new;
}

// `filled_dev` != NULL: the fill count lives in device memory; it is read by the append launch and advanced by a
// second, one-thread launch behind it (`filled` is then ignored).
int cache_append(const void* k_new, const void* v_new, void* K, void* V, void* Kc, void* Vc, void* Kb, int B, int Hkv, int D,
                 int t_new, int filled, int32_t* filled_dev, int max_len, int nc_alloc, int nb_alloc, int cblock, int cstride,
                 int sblock, int dtype, cudaStream_t st) {
  NSA_REQUIRE(D % 8 == 0 && D > 0, NSA_ERR_ARG, "cache append: D %d must be a positive multiple of 8", D);
  if (filled_dev != nullptr) filled = 0;
  NSA_REQUIRE(t_new >= 0 && filled >= 0 && filled + t_new <= max_len, NSA_ERR_ARG,
              "cache append: %d filled + %d new rows exceed the allocation of %d", filled, t_new, max_len);
  NSA_REQUIRE(cblock > 0 && cstride > 0 && cstride <= cblock && sblock > 0, NSA_ERR_ARG, "cache append: bad block sizes");
  NSA_REQUIRE((long long)B * Hkv <= 65535 && B * Hkv > 0, NSA_ERR_ARG, "cache append: B*Hkv %lld", (long long)B * Hkv);
  if (t_new == 0) return NSA_OK;
  const int T0 = filled, T1 = filled + t_new;
  auto n_pooled = [&](int len) { return cstride == cblock ? (len + cblock - 1) / cblock : (len >= cblock ? (len - cblock) / cstride + 1 : 0); };
  // windows that contain a new row: whole windows completed by them, or (stride == block) the partial tail window
  int c0 = cstride == cblock ? T0 / cblock : n_pooled(T0);
  int nw = n_pooled(T1) - c0;
  int b0 = T0 / sblock, nbk = (T1 + sblock - 1) / sblock - b0;
  if (filled_dev != nullptr) {                             // the most windows / blocks t_new rows can touch at any fill count
    nw = (t_new + cstride - 1) / cstride + 1;
    nbk = (t_new + sblock - 1) / sblock + 1;
  } else {
    NSA_REQUIRE(c0 + nw <= nc_alloc && b0 + nbk <= nb_alloc, NSA_ERR_ARG, "cache append: pooled (%d) or block-mean (%d) allocation too small",
                nc_alloc, nb_alloc);
  }
  const long long threads = ((long long)t_new + nw + nbk) * (D / 8);
  dim3 grid((unsigned)((threads + 255) / 256), (unsigned)(B * Hkv));
#define NSA_APPEND(TT)                                                                                                  \
  cache_append_kernel<TT><<<grid, 256, 0, st>>>((const TT*)k_new, (const TT*)v_new, (TT*)K, (TT*)V, (TT*)Kc, (TT*)Vc, (TT*)Kb, D, \
                                                t_new, filled, max_len, nc_alloc, nb_alloc, cblock, cstride, c0, nw, sblock, b0, nbk, filled_dev)
  if (dtype == NSA_BF16) NSA_APPEND(__nv_bfloat16);
  else if (dtype == NSA_FP16) NSA_APPEND(__half);
  else return fail(NSA_ERR_UNSUPPORTED, "cache append: dtype %d", dtype);
#undef NSA_APPEND
  if (filled_dev != nullptr) cache_advance_kernel<<<1, 32, 0, st>>>(filled_dev, t_new, max_len);
  return launch_status("cache_append");
}

// ------------------------------------------------------------------ top-k over one score row
// Warp-level: k_out rounds of (lane-local scan, shuffle arg-max).  Order: larger score
// first, equal scores lowest index first.  Chosen entries are overwritten with a quiet-NaN
// marker that no finite/inf score equals.
__device__ __forceinline__ bool better(float v, int c, float bv, int bc) { return v > bv || (v == bv && c < bc); }

// (value, index) arg-max over the warp in two redux instructions: scores map to unsigned keys that keep their
// order (a lane without a candidate holds key 0, below every real score), the largest key wins, and among the
// lanes holding it the lowest index.
__device__ __forceinline__ uint32_t order_key(float v) {
  const uint32_t u = __float_as_uint(v + 0.f);             // -0 and +0 compare equal: both become +0
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ int warp_argmax(float v, int c, int none) {
  const uint32_t key = c == none ? 0u : order_key(v);
  const uint32_t best = __reduce_max_sync(0xffffffffu, key);
  return (int)__reduce_min_sync(0xffffffffu, (uint32_t)((key == best && c != none) ? c : none));
}

__device__ void warp_topk_row(float* s, int n_scan, int nk, int k_out, int32_t* out_row, int lane) {
  const uint32_t TAKEN = 0xFFFFFFFFu;
  const int NONE = 0x7fffffff;
  const int n_pick = min(k_out, n_scan);
  // Lane L owns the elements L, L+32, L+64, ... and remembers the best of them.  A round picks the best of the 32
  // remembered candidates; only the owner of the picked element needs a new candidate, and the whole warp
  // finds it: one strided element per lane, another warp arg-max.
  float bv = -INFINITY;
  int bc = NONE;
#pragma unroll 4
  for (int c = lane; c < n_scan; c += 32) {
    const float v = s[c];
    if (bc == NONE || v > bv) { bv = v; bc = c; }
  }
  int picked = n_pick;
  for (int it = 0; it < n_pick; ++it) {
    const int gc = warp_argmax(bv, bc, NONE);
    // no candidate left: caller-supplied scores may carry the bit pattern that marks a taken entry (an all-ones NaN);
    // such entries are never offered, so fewer than n_pick can be picked -- the rest is filled like the tail below
    if (gc == NONE) { picked = it; break; }
    if (lane == 0) { out_row[it] = gc; s[gc] = __uint_as_float(TAKEN); }
    __syncwarp();
    const int owner = gc & 31;
    float rv = -INFINITY;
    int rc = NONE;
    for (int c = owner + 32 * lane; c < n_scan; c += 32 * 32) {
      const float v = s[c];
      if (__float_as_uint(v) != TAKEN && (rc == NONE || better(v, c, rv, rc))) { rv = v; rc = c; }
    }
    const int nc = warp_argmax(rv, rc, NONE);
    if (lane == owner) { bc = nc; bv = nc == NONE ? -INFINITY : s[nc]; }
  }
  // fewer candidates than slots: the remaining slots take the lowest block ids not scanned
  for (int it = picked + lane; it < k_out; it += 32) out_row[it] = n_scan + (it - picked);
  (void)nk;
}

// ------------------------------------------------------------------ score + select
// Thread block = (batch, index head, chunk of R query blocks); warp w owns query block row w.
// An index head is a query head (GS = 1) or, for indices shared by a GQA group, a KV head; its query
// vector is then the fp32 sum, in head order, of the block means of its GS = H/Hkv query heads (the
// score of the group is the dot of that sum with the K block mean -- GS times less work than summing
// per-head dots, and the definition the CPU oracle restates).
// Kb tiles of 64 block-means are staged in shared memory once per chunk and shared by the rows.
// ------------------------------------------------------------------ MoBA routing
// A second producer of block lists: every query TOKEN picks its top_kq key blocks by q . mean(K block) * scale;
// a query block lists the union of its rows' picks.  One thread block per (query block, batch*head), one warp per
// row at a time: lane = key block, fp32 fma over D in index order against the block means (L1/L2 resident), the row's
// scores in shared memory, picks by the same warp arg-max rounds as the other selections (ties -> lowest id).  The
// union is a bit set; the best score any row gave a block (for the overflow rule) an order-preserving integer max.
template <typename T>
__global__ void __launch_bounds__(256) moba_route_kernel(const T* __restrict__ Q, const T* __restrict__ Kb, int32_t* __restrict__ idx,
                                                         int H, int Hkv, int Tq, int nq, int nk, int D, int kq, int cap, int bm, int bn,
                                                         int offset, int causal, float scale) {
  extern __shared__ unsigned char moba_smem[];
  const int nkp = (nk + 31) & ~31;
  float* sc = reinterpret_cast<float*>(moba_smem);                  // [8][nkp] one score row per warp
  uint32_t* level = reinterpret_cast<uint32_t*>(sc + 8 * nkp);       // [nkp] order keys of the block-level maxima
  uint32_t* bits = level + nkp;                                      // [nkp/32] union of the picks
  int32_t* picks = reinterpret_cast<int32_t*>(bits + nkp / 32);      // [8][64]
  float* qrow = reinterpret_cast<float*>(picks + 8 * 64);            // [8][D]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qb = blockIdx.x, bh = blockIdx.y;
  const int b = bh / H, h = bh % H;
  const int hk = h / (H / Hkv);
  const T* Kh = Kb + ((size_t)b * Hkv + hk) * nk * D;
  for (int i = threadIdx.x; i < nkp; i += 256) level[i] = 0u;
  for (int i = threadIdx.x; i < nkp / 32; i += 256) bits[i] = 0u;
  __syncthreads();
  float* my = sc + warp * nkp;
  float* myq = qrow + warp * D;
  for (int r = warp; r < bm; r += 8) {
    const int row = qb * bm + r;
    // the query row as fp32 (rows past the end are the zero rows of the padded tensor)
    for (int d = lane; d < D; d += 32) myq[d] = row < Tq ? Elem<T>::to_f(Q[((size_t)bh * Tq + row) * D + d]) : 0.f;
    __syncwarp();
    int n_legal = nk;
    if (causal) {
      const long long lim = (long long)row + offset;
      n_legal = lim < 0 ? 0 : (int)min((long long)nk, lim / bn + 1);
    }
    for (int n = lane; n < n_legal; n += 32) {
      const T* kr = Kh + (size_t)n * D;
      float acc = 0.f;
      for (int d8 = 0; d8 < D; d8 += 8) {
        const uint4 raw = *reinterpret_cast<const uint4*>(kr + d8);
        const uint32_t* w = reinterpret_cast<const uint32_t*>(&raw);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = Elem<T>::unpack(w[e]);
          acc = fmaf(myq[d8 + 2 * e], f.x, acc);
          acc = fmaf(myq[d8 + 2 * e + 1], f.y, acc);
        }
      }
      const float v = acc * scale;
      my[n] = v;
      atomicMax(&level[n], order_key(v));
    }
    __syncwarp();
    const int n_pick = min(kq, n_legal);
    if (n_pick > 0) {
      warp_topk_row(my, n_legal, nk, n_pick, picks + warp * 64, lane);
      __syncwarp();
      for (int i = lane; i < n_pick; i += 32) {
        const int c = picks[warp * 64 + i];
        if (c >= 0 && c < n_legal) atomicOr(&bits[c >> 5], 1u << (c & 31));
      }
    }
    __syncwarp();
  }
  __syncthreads();
  if (warp != 0) return;
  int32_t* out = idx + ((size_t)bh * nq + qb) * cap;
  int total = 0;
  for (int w0 = lane; w0 < nkp / 32; w0 += 32) total += __popc(bits[w0]);
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) total += __shfl_xor_sync(0xffffffffu, total, d);
  if (total <= cap) {
    // ascending ids, then the out-of-range id nk
    int pos = 0;
    for (int w0 = 0; w0 < nkp / 32; ++w0) {
      const uint32_t word = bits[w0];
      if ((word >> lane) & 1u) out[pos + __popc(word & ((1u << lane) - 1))] = w0 * 32 + lane;
      pos += __popc(word);
    }
    for (int i = pos + lane; i < cap; i += 32) out[i] = nk;
  } else {
    // more distinct blocks than slots: keep the cap with the best block-level score, best first
    float* lv = sc;
    for (int n = lane; n < nk; n += 32) {
      const uint32_t k = level[n];
      const uint32_t u = (k & 0x80000000u) ? (k & 0x7fffffffu) : ~k;         // inverse of order_key
      lv[n] = ((bits[n >> 5] >> (n & 31)) & 1u) ? __uint_as_float(u) : -INFINITY;
    }
    __syncwarp();
    warp_topk_row(lv, nk, nk, cap, out, lane);
  }
}

int moba_route(const void* Q, const void* Kb, int32_t* idx, int B, int H, int Hkv, int Tq, int nq, int nk, int D, int kq, int cap,
               int bm, int bn, int offset, int causal, float scale, int dtype, cudaStream_t st) {
  NSA_REQUIRE(B > 0 && H > 0 && Hkv > 0 && H % Hkv == 0 && Tq > 0 && nq == (Tq + bm - 1) / bm && nk > 0, NSA_ERR_ARG, "moba routing: sizes");
  NSA_REQUIRE(D % 8 == 0 && D > 0 && bm > 0 && bn > 0, NSA_ERR_ARG, "moba routing: D %d must be a positive multiple of 8", D);
  NSA_REQUIRE(kq >= 1 && kq <= 64, NSA_ERR_UNSUPPORTED, "moba routing: top_k_per_query %d not in [1, 64]", kq);
  NSA_REQUIRE(cap >= 1 && cap <= nk, NSA_ERR_ARG, "moba routing: cap %d must be in [1, nk = %d]", cap, nk);
  NSA_REQUIRE((long long)B * H <= 65535, NSA_ERR_ARG, "moba routing: B*H too large");
  const int nkp = (nk + 31) & ~31;
  const size_t smem = (size_t)8 * nkp * 4 + (size_t)nkp * 4 + nkp / 8 + 8 * 64 * 4 + (size_t)8 * D * 4;
  NSA_REQUIRE(smem <= 200 * 1024, NSA_ERR_UNSUPPORTED, "moba routing: %d key blocks do not fit shared memory", nk);
  dim3 grid((unsigned)nq, (unsigned)(B * H));
#define NSA_MOBA(TT)                                                                                                   \
  {                                                                                                                     \
    auto fn = moba_route_kernel<TT>;                                                                                    \
    NSA_CUDA_OK(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));                     \
    fn<<<grid, 256, smem, st>>>((const TT*)Q, (const TT*)Kb, idx, H, Hkv, Tq, nq, nk, D, kq, cap, bm, bn, offset, causal, scale); \
  }
  if (dtype == NSA_BF16) NSA_MOBA(__nv_bfloat16)
  else if (dtype == NSA_FP16) NSA_MOBA(__half)
  else return fail(NSA_ERR_UNSUPPORTED, "moba routing: dtype %d", dtype);
#undef NSA_MOBA
  return launch_status("moba_route");
}

template <typename T, int D>
__global__ void __launch_bounds__(256) select_blocks_kernel(const T* __restrict__ Qb, const T* __restrict__ Kb,
                                                            int32_t* __restrict__ idx, int H, int Hkv, int Hi, int nq, int nk,
                                                            int k_out, int bm, int bn, int offset, int causal, float scale,
                                                            int force_first, int force_local, int R,
                                                            const int32_t* __restrict__ dyn_len) {
  constexpr int KT = 64;
  // key length in device memory (decoding under a captured graph): the padded-length offset of the block grid
  if (dyn_len != nullptr) offset = (*dyn_len + bn - 1) / bn * bn - ((nq * bm + bm - 1) / bm) * bm;
  constexpr int PITCH = D + 8;     // 16-bit elements; 16-byte aligned rows, 17-chunk stride -> conflict-free 128-bit reads
  // The block's 8 warps cover R query blocks x CW = 8/R tiles of 64 key blocks at a time: with many query
  // blocks R = 8 and a warp owns a row; with few (decoding: one) the warps share a row and take different key
  // tiles.  A score is always one lane's fma chain over D in index order, whichever warp computes it.
  const int CW = 8 / R;
  extern __shared__ __align__(16) unsigned char smem[];
  T* kt = reinterpret_cast<T*>(smem);                              // [CW*KT][PITCH]
  const int G = H / Hkv;
  const int GS = Hi == H ? 1 : G;                                  // query heads summed per index head
  float* qs = reinterpret_cast<float*>(kt + CW * KT * PITCH);      // [R][D] fp32 query vectors
  float* sc = qs + R * D;                                          // [R][nk]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int wrow = warp % R, wslot = warp / R;                     // row of the block / key tile of the group
  const int bh = blockIdx.y, b = bh / Hi, hi = bh % Hi;
  const int hk = Hi == H ? hi / G : hi;
  const int h0 = Hi == H ? hi : hi * G;                            // first query head of this index head
  const int qb0 = blockIdx.x * R;
  const int rows = min(R, nq - qb0);
  const T* kbase = Kb + ((size_t)(b * Hkv + hk) * nk) * D;

  for (int i = threadIdx.x; i < rows * D; i += blockDim.x) {
    const int r = i / D, d = i % D;
    // sum over the group's heads in head order; the loads of a batch of 8 heads are issued together
    float acc = 0.f;
    for (int g0 = 0; g0 < GS; g0 += 8) {
      float v[8];
#pragma unroll
      for (int e = 0; e < 8; ++e)
        v[e] = g0 + e < GS ? Elem<T>::to_f(Qb[(((size_t)b * H + h0 + g0 + e) * nq + qb0 + r) * D + d]) : 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e)
        if (g0 + e < GS) acc = (g0 + e == 0) ? v[e] : __fadd_rn(acc, v[e]);
    }
    qs[i] = acc;
  }

  // legal range per row: blocks 0..cmax
  auto cmax_of = [&](int qb) {
    if (!causal) return nk - 1;
    long long last = (long long)qb * bm + (bm - 1) + offset;
    if (last < 0) return -1;
    return (int)min((long long)(nk - 1), last / bn);
  };
  const int cmax_chunk = cmax_of(qb0 + rows - 1);
  const int my_qb = qb0 + wrow;
  const int my_cmax = wrow < rows ? cmax_of(my_qb) : -1;
  float* my_sc = sc + (size_t)wrow * nk;

  for (int c0 = 0; c0 <= cmax_chunk; c0 += KT * CW) {
    __syncthreads();
    const int nrow = min(KT * CW, nk - c0);
    // asynchronous 16-byte copies, all in flight at once (a load-then-store loop pays one memory round trip per
    // iteration, which is what a launch with a handful of thread blocks -- decoding -- would wait on)
    for (int i = threadIdx.x; i < KT * CW * (D / 8); i += blockDim.x) {
      const int r = i / (D / 8), w = i % (D / 8);
      const bool in = r < nrow;
      cp_async16(smem_u32(kt + r * PITCH + w * 8), kbase + (size_t)(c0 + (in ? r : 0)) * D + w * 8, in ? 16 : 0);
    }
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();
    const int cw0 = c0 + wslot * KT;                               // this warp's tile of key blocks
    if (wrow < rows && cw0 <= my_cmax) {
      // lane owns blocks cw0+lane and cw0+lane+32: two independent fma chains in index order
      const uint4* k0 = reinterpret_cast<const uint4*>(kt + (wslot * KT + lane) * PITCH);
      const uint4* k1 = reinterpret_cast<const uint4*>(kt + (wslot * KT + lane + 32) * PITCH);
      const float4* qv = reinterpret_cast<const float4*>(qs + wrow * D);
      float tot0 = 0.f, tot1 = 0.f;
#pragma unroll 4
      for (int w = 0; w < D / 8; ++w) {
        const uint4 kv0 = k0[w], kv1 = k1[w];
        const float4 qa = qv[2 * w], qb_ = qv[2 * w + 1];
        const float q[8] = {qa.x, qa.y, qa.z, qa.w, qb_.x, qb_.y, qb_.z, qb_.w};
        const uint32_t kw0[4] = {kv0.x, kv0.y, kv0.z, kv0.w}, kw1[4] = {kv1.x, kv1.y, kv1.z, kv1.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f0 = Elem<T>::unpack(kw0[e]), f1 = Elem<T>::unpack(kw1[e]);
          tot0 = __fmaf_rn(q[2 * e], f0.x, tot0);
          tot0 = __fmaf_rn(q[2 * e + 1], f0.y, tot0);
          tot1 = __fmaf_rn(q[2 * e], f1.x, tot1);
          tot1 = __fmaf_rn(q[2 * e + 1], f1.y, tot1);
        }
      }
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int c = cw0 + lane + half * 32;
        if (c < nk && c <= my_cmax) {
          float v = (half == 0 ? tot0 : tot1) * scale;
          if (c < force_first || c > my_cmax - force_local) v = INFINITY;
          my_sc[c] = v;
        }
      }
    }
  }
  __syncthreads();                                                 // a row's scores come from several warps
  if (wrow < rows && wslot == 0) {
    int32_t* out_row = idx + ((size_t)bh * nq + my_qb) * k_out;
    warp_topk_row(my_sc, my_cmax + 1, nk, k_out, out_row, lane);
  }
}

template <typename T>
static int select_launch(const void* Qb, const void* Kb, int32_t* idx, int B, int H, int Hkv, int Hi, int nq, int nk, int D,
                         int k_out, int bm, int bn, int offset, int causal, float scale, int ff, int fl, const int32_t* dyn_len,
                         cudaStream_t st) {
  // R query blocks per thread block (a power of two <= 8): no more than there are, fewer if the score rows
  // would not fit; the other 8/R warps of a row group take further key tiles
  int R = 8;
  while (R > 1 && R / 2 >= nq) R >>= 1;
  auto need = [&](int r) { return (size_t)(8 / r) * 64 * (D + 8) * 2 + (size_t)r * D * 4 + (size_t)r * nk * 4; };
  while (R > 1 && need(R) > 200 * 1024) R >>= 1;
  NSA_REQUIRE(need(R) <= 200 * 1024, NSA_ERR_UNSUPPORTED, "select: %d KV blocks exceed the shared-memory score row", nk);
  dim3 grid((unsigned)((nq + R - 1) / R), (unsigned)(B * Hi));
  size_t smem = need(R);
#define NSA_SEL(DD)                                                                                     \
  {                                                                                                     \
    auto fn = select_blocks_kernel<T, DD>;                                                              \
    NSA_CUDA_OK(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));      \
    fn<<<grid, 256, smem, st>>>((const T*)Qb, (const T*)Kb, idx, H, Hkv, Hi, nq, nk, k_out, bm, bn, offset, \
                                causal, scale, ff, fl, R, dyn_len);                                     \
  }
  switch (D) {
    case 32: NSA_SEL(32) break;
    case 64: NSA_SEL(64) break;
    case 128: NSA_SEL(128) break;
    default: return fail(NSA_ERR_UNSUPPORTED, "select: head dim %d not in {32,64,128}", D);
  }
#undef NSA_SEL
  return launch_status("select_blocks");
}

int select_blocks(const void* Qb, const void* Kb, int32_t* idx, int B, int H, int Hkv, int nq, int nk, int D, int top_k,
                  int bm, int bn, int offset, int causal, float scale, int ff, int fl, int shared, int dtype,
                  const int32_t* dyn_len, cudaStream_t st) {
  const int Hi = shared ? Hkv : H;
  NSA_REQUIRE(B > 0 && H > 0 && Hkv > 0 && H % Hkv == 0, NSA_ERR_ARG, "select: heads %d/%d", H, Hkv);
  NSA_REQUIRE(nq > 0 && nk > 0 && top_k > 0 && bm > 0 && bn > 0, NSA_ERR_ARG, "select: empty problem");
  NSA_REQUIRE((long long)B * H <= 65535, NSA_ERR_ARG, "select: B*H too large");
  NSA_REQUIRE(ff >= 0 && fl >= 0, NSA_ERR_ARG, "select: negative forced-block counts");
  int k_out = top_k < nk ? top_k : nk;
  if (dtype == NSA_BF16)
    return select_launch<__nv_bfloat16>(Qb, Kb, idx, B, H, Hkv, Hi, nq, nk, D, k_out, bm, bn, offset, causal, scale, ff, fl, dyn_len, st);
  if (dtype == NSA_FP16)
    return select_launch<__half>(Qb, Kb, idx, B, H, Hkv, Hi, nq, nk, D, k_out, bm, bn, offset, causal, scale, ff, fl, dyn_len, st);
  return fail(NSA_ERR_UNSUPPORTED, "select: dtype %d", dtype);
}

// ------------------------------------------------------------------ top-k from given scores
__global__ void __launch_bounds__(256) topk_scores_kernel(const float* __restrict__ scores, int32_t* __restrict__ idx,
                                                          int nq, int nk, int k_out, int bm, int bn, int offset,
                                                          int causal, int R) {
  extern __shared__ __align__(16) unsigned char smem[];
  float* sc = reinterpret_cast<float*>(smem);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bh = blockIdx.y;
  const int qb = blockIdx.x * R + warp;
  if (warp >= R || qb >= nq) return;
  int cmax = nk - 1;
  if (causal) {
    long long last = (long long)qb * bm + (bm - 1) + offset;
    cmax = last < 0 ? -1 : (int)min((long long)(nk - 1), last / bn);
  }
  float* my = sc + (size_t)warp * nk;
  const float* src = scores + ((size_t)bh * nq + qb) * nk;
  for (int c = lane; c <= cmax; c += 32) my[c] = src[c];
  __syncwarp();
  warp_topk_row(my, cmax + 1, nk, k_out, idx + ((size_t)bh * nq + qb) * k_out, lane);
}

int topk_from_scores(const float* scores, int32_t* idx, int BH, int nq, int nk, int top_k, int bm, int bn, int offset,
                     int causal, cudaStream_t st) {
  NSA_REQUIRE(BH > 0 && nq > 0 && nk > 0 && top_k > 0, NSA_ERR_ARG, "topk: empty problem");
  NSA_REQUIRE(BH <= 65535, NSA_ERR_ARG, "topk: B*H too large");
  int R = 8;
  while (R > 1 && (size_t)R * nk * 4 > 200 * 1024) R >>= 1;
  NSA_REQUIRE((size_t)R * nk * 4 <= 200 * 1024, NSA_ERR_UNSUPPORTED, "topk: %d KV blocks exceed shared memory", nk);
  size_t smem = (size_t)R * nk * 4;
  NSA_CUDA_OK(cudaFuncSetAttribute(topk_scores_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid((unsigned)((nq + R - 1) / R), (unsigned)BH);
  topk_scores_kernel<<<grid, 256, smem, st>>>(scores, idx, nq, nk, top_k < nk ? top_k : nk, bm, bn, offset, causal, R);
  return launch_status("topk_from_scores");
}

}  // namespace nsa
