// HBM-bound element-wise kernels: gated combine, fp8 absmax / quantise, the backward's
// delta pre-pass, the fp32 -> 16-bit gradient cast and the rotary-embedding + head-major re-layout
// of the projection outputs.  All use 128-bit accesses and a
// grid-stride loop sized to a multiple of the SM count.
#include "common.cuh"

namespace nsa {

static int grid_for(long long work_items, int threads) {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  long long want = (work_items + threads - 1) / threads;
  long long cap = (long long)sms * 16;
  return (int)(want < 1 ? 1 : (want < cap ? want : cap));
}

__device__ __forceinline__ float load_any(const void* p, size_t i, int dt) {
  if (dt == NSA_FP32) return reinterpret_cast<const float*>(p)[i];
  if (dt == NSA_FP16) return __half2float(reinterpret_cast<const __half*>(p)[i]);
  return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}
__device__ __forceinline__ float round_to(float x, int dt) {
  if (dt == NSA_FP16) return __half2float(__float2half_rn(x));
  if (dt == NSA_BF16) return __bfloat162float(__float2bfloat16_rn(x));
  return x;
}

// ------------------------------------------------------------------ combine
// One thread = 8 consecutive columns of one row.
template <typename T>
__global__ void __launch_bounds__(256) combine16_kernel(const T* __restrict__ oc, const T* __restrict__ os,
                                                        const T* __restrict__ ow, const void* __restrict__ gates,
                                                        void* __restrict__ out, long long rows, int D, int act,
                                                        int dt, int gdt) {
  const int CH = D / 8;
  const long long total = rows * CH;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / CH;
    const int ch = (int)(i % CH);
    float x0 = load_any(gates, r * 3 + 0, gdt), x1 = load_any(gates, r * 3 + 1, gdt), x2 = load_any(gates, r * 3 + 2, gdt);
    float g0, g1, g2;
    if (act == NSA_GATE_SOFTMAX) {
      float mx = fmaxf(x0, fmaxf(x1, x2));
      float e0 = expf(x0 - mx), e1 = expf(x1 - mx), e2 = expf(x2 - mx);
      float s = e0 + e1 + e2;
      g0 = e0 / s; g1 = e1 / s; g2 = e2 / s;
    } else {
      g0 = 1.f / (1.f + expf(-x0)); g1 = 1.f / (1.f + expf(-x1)); g2 = 1.f / (1.f + expf(-x2));
    }
    const size_t e0i = (size_t)r * D + ch * 8;
    uint4 a = *reinterpret_cast<const uint4*>(oc + e0i);
    uint4 b = *reinterpret_cast<const uint4*>(os + e0i);
    uint4 c = *reinterpret_cast<const uint4*>(ow + e0i);
    const uint32_t* aw = reinterpret_cast<const uint32_t*>(&a);
    const uint32_t* bw = reinterpret_cast<const uint32_t*>(&b);
    const uint32_t* cw = reinterpret_cast<const uint32_t*>(&c);
    if (gdt != NSA_FP32) {
      // 16-bit gates: every intermediate is rounded to the 16-bit type, left to right
      g0 = round_to(g0, dt); g1 = round_to(g1, dt); g2 = round_to(g2, dt);
      uint32_t w[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float2 fa = Elem<T>::unpack(aw[e]), fb = Elem<T>::unpack(bw[e]), fc = Elem<T>::unpack(cw[e]);
        float lo = round_to(round_to(round_to(g0 * fa.x, dt) + round_to(g1 * fb.x, dt), dt) + round_to(g2 * fc.x, dt), dt);
        float hi = round_to(round_to(round_to(g0 * fa.y, dt) + round_to(g1 * fb.y, dt), dt) + round_to(g2 * fc.y, dt), dt);
        w[e] = Elem<T>::pack(lo, hi);
      }
      *reinterpret_cast<uint4*>(reinterpret_cast<T*>(out) + e0i) = make_uint4(w[0], w[1], w[2], w[3]);
    } else {
      float o[8];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float2 fa = Elem<T>::unpack(aw[e]), fb = Elem<T>::unpack(bw[e]), fc = Elem<T>::unpack(cw[e]);
        o[2 * e] = (g0 * fa.x + g1 * fb.x) + g2 * fc.x;
        o[2 * e + 1] = (g0 * fa.y + g1 * fb.y) + g2 * fc.y;
      }
      float4* q = reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + e0i);
      q[0] = make_float4(o[0], o[1], o[2], o[3]);
      q[1] = make_float4(o[4], o[5], o[6], o[7]);
    }
  }
}

int combine(const void* oc, const void* os, const void* ow, const void* gates, void* out, long long rows, int D,
            int act, int dtype, int gate_dtype, cudaStream_t st) {
  NSA_REQUIRE(D > 0 && D % 8 == 0, NSA_ERR_ARG, "combine: D %d must be a multiple of 8", D);
  NSA_REQUIRE(act == NSA_GATE_SIGMOID || act == NSA_GATE_SOFTMAX, NSA_ERR_ARG, "combine: activation %d", act);
  NSA_REQUIRE(gate_dtype == dtype || gate_dtype == NSA_FP32, NSA_ERR_UNSUPPORTED,
              "combine: gate dtype %d with branch dtype %d", gate_dtype, dtype);
  if (rows == 0) return NSA_OK;
  int grid = grid_for(rows * (D / 8), 256);
  if (dtype == NSA_BF16)
    combine16_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)oc, (const __nv_bfloat16*)os,
                                                          (const __nv_bfloat16*)ow, gates, out, rows, D, act, dtype, gate_dtype);
  else if (dtype == NSA_FP16)
    combine16_kernel<__half><<<grid, 256, 0, st>>>((const __half*)oc, (const __half*)os, (const __half*)ow, gates, out,
                                                   rows, D, act, dtype, gate_dtype);
  else
    return fail(NSA_ERR_UNSUPPORTED, "combine: dtype %d", dtype);
  return launch_status("combine");
}

// ------------------------------------------------------------------ fp8 absmax / quantise
__global__ void __launch_bounds__(256) absmax_kernel(const void* __restrict__ x, long long n, int dt, float* __restrict__ out) {
  float m = 0.f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    m = fmaxf(m, fabsf(load_any(x, (size_t)i, dt)));
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
  __shared__ float wm[8];
  if ((threadIdx.x & 31) == 0) wm[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; ++w) m = fmaxf(m, wm[w]);
    atomicMax(reinterpret_cast<int*>(out), __float_as_int(m));   // non-negative floats order like ints
  }
}

int fp8_absmax(const void* x, long long n, int dtype, float* absmax, cudaStream_t st) {
  NSA_REQUIRE(dtype == NSA_BF16 || dtype == NSA_FP16 || dtype == NSA_FP32, NSA_ERR_UNSUPPORTED, "absmax: dtype %d", dtype);
  if (n == 0) return NSA_OK;
  absmax_kernel<<<grid_for(n, 256), 256, 0, st>>>(x, n, dtype, absmax);
  return launch_status("fp8_absmax");
}

__global__ void __launch_bounds__(256) quantize_kernel(const void* __restrict__ x, uint8_t* __restrict__ out, long long n,
                                                       int dt, int fmt, float scale, float fmax) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    float q = round_to(__fdiv_rn(load_any(x, (size_t)i, dt), scale), dt);
    q = fminf(fmaxf(q, -fmax), fmax);
    out[i] = (uint8_t)__nv_cvt_float_to_fp8(q, __NV_SATFINITE, fmt == NSA_FP8_E5M2 ? __NV_E5M2 : __NV_E4M3);
  }
}

int fp8_quantize(const void* x, void* out8, long long n, int dtype, int fmt, float scale, cudaStream_t st) {
  NSA_REQUIRE(dtype == NSA_BF16 || dtype == NSA_FP16 || dtype == NSA_FP32, NSA_ERR_UNSUPPORTED, "quantize: dtype %d", dtype);
  NSA_REQUIRE(fmt == NSA_FP8_E4M3 || fmt == NSA_FP8_E5M2, NSA_ERR_ARG, "quantize: format %d", fmt);
  NSA_REQUIRE(scale > 0.f, NSA_ERR_ARG, "quantize: scale must be positive");
  if (n == 0) return NSA_OK;
  quantize_kernel<<<grid_for(n, 256), 256, 0, st>>>(x, (uint8_t*)out8, n, dtype, fmt, scale,
                                                    fmt == NSA_FP8_E5M2 ? 57344.f : 448.f);
  return launch_status("fp8_quantize");
}

// out[i] = bf16(fp32(x8[i]) * scale): 16 elements (one 16-byte load, two 16-byte stores) per thread and step
__global__ void __launch_bounds__(256) dequantize_kernel(const uint8_t* __restrict__ x, __nv_bfloat16* __restrict__ out,
                                                         long long n, int fmt, float scale) {
  const long long nvec = n / 16;
  for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < nvec; v += (long long)gridDim.x * blockDim.x) {
    const uint4 raw = reinterpret_cast<const uint4*>(x)[v];
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
    uint32_t o[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const uint32_t two = (w[e >> 1] >> ((e & 1) * 16)) & 0xffffu;
      o[e] = Elem<__nv_bfloat16>::pack(fp8_to_f((uint8_t)(two & 0xffu), fmt) * scale, fp8_to_f((uint8_t)(two >> 8), fmt) * scale);
    }
    uint4* dst = reinterpret_cast<uint4*>(out) + 2 * v;
    dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
    dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
  }
  // ragged tail (n not a multiple of 16)
  for (long long i = nvec * 16 + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    out[i] = __float2bfloat16_rn(fp8_to_f(x[i], fmt) * scale);
}

int fp8_dequantize(const void* x8, void* out, long long n, int fmt, float scale, cudaStream_t st) {
  NSA_REQUIRE(fmt == NSA_FP8_E4M3 || fmt == NSA_FP8_E5M2, NSA_ERR_ARG, "dequantize: format %d", fmt);
  NSA_REQUIRE(scale > 0.f, NSA_ERR_ARG, "dequantize: scale must be positive");
  NSA_REQUIRE((reinterpret_cast<uintptr_t>(x8) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0, NSA_ERR_ARG,
              "dequantize: pointers must be 16-byte aligned");
  if (n == 0) return NSA_OK;
  dequantize_kernel<<<grid_for((n + 15) / 16, 256), 256, 0, st>>>((const uint8_t*)x8, (__nv_bfloat16*)out, n, fmt, scale);
  return launch_status("fp8_dequantize");
}

// ------------------------------------------------------------------ backward helpers
// delta[r] = sum_d dO[r,d]*O[r,d]; one warp per row, 16-byte loads.
template <typename T>
__global__ void __launch_bounds__(256) delta_kernel(const T* __restrict__ dO, const T* __restrict__ O, float* __restrict__ delta,
                                                    long long rows, int D) {
  const int lane = threadIdx.x & 31;
  const int CH = D / 8;
  for (long long r = (long long)blockIdx.x * 8 + (threadIdx.x >> 5); r < rows; r += (long long)gridDim.x * 8) {
    float acc = 0.f;
    for (int ch = lane; ch < CH; ch += 32) {
      uint4 a = *reinterpret_cast<const uint4*>(dO + (size_t)r * D + ch * 8);
      uint4 b = *reinterpret_cast<const uint4*>(O + (size_t)r * D + ch * 8);
      const uint32_t* aw = reinterpret_cast<const uint32_t*>(&a);
      const uint32_t* bw = reinterpret_cast<const uint32_t*>(&b);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float2 fa = Elem<T>::unpack(aw[e]), fb = Elem<T>::unpack(bw[e]);
        acc = fmaf(fa.x, fb.x, acc);
        acc = fmaf(fa.y, fb.y, acc);
      }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    if (lane == 0) delta[r] = acc;
  }
}

int bwd_delta(const void* dO, const void* O, float* delta, long long rows, int D, int dtype, cudaStream_t st) {
  NSA_REQUIRE(D > 0 && D % 8 == 0, NSA_ERR_ARG, "delta: D %d must be a multiple of 8", D);
  if (rows == 0) return NSA_OK;
  int grid = grid_for(rows * 32, 256);
  if (dtype == NSA_BF16) delta_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)dO, (const __nv_bfloat16*)O, delta, rows, D);
  else if (dtype == NSA_FP16) delta_kernel<__half><<<grid, 256, 0, st>>>((const __half*)dO, (const __half*)O, delta, rows, D);
  else return fail(NSA_ERR_UNSUPPORTED, "delta: dtype %d", dtype);
  return launch_status("bwd_delta");
}

template <typename T>
__global__ void __launch_bounds__(256) cast_kernel(const float* __restrict__ src, T* __restrict__ dst, long long n) {
  const long long n4 = n / 4;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    float4 v = reinterpret_cast<const float4*>(src)[i];
    uint2 w = make_uint2(Elem<T>::pack(v.x, v.y), Elem<T>::pack(v.z, v.w));
    reinterpret_cast<uint2*>(dst)[i] = w;
  }
  if (blockIdx.x == 0)
    for (long long i = n4 * 4 + threadIdx.x; i < n; i += blockDim.x) dst[i] = Elem<T>::from_f(src[i]);
}

int cast_from_f32(const float* src, void* dst, long long n, int dtype, cudaStream_t st) {
  if (n == 0) return NSA_OK;
  int grid = grid_for(n / 4 + 1, 256);
  if (dtype == NSA_BF16) cast_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(src, (__nv_bfloat16*)dst, n);
  else if (dtype == NSA_FP16) cast_kernel<__half><<<grid, 256, 0, st>>>(src, (__half*)dst, n);
  else return fail(NSA_ERR_UNSUPPORTED, "cast: dtype %d", dtype);
  return launch_status("cast_from_f32");
}

// ------------------------------------------------------------------ rotary embedding + [B,T,H,D] -> [B,H,T,D]
// One thread = 8 consecutive columns d0..d0+7 of the first half of a row AND their partners d0+D/2..:
// out[d] = x[d] cos[d] - x[d+D/2] sin[d],  out[d+D/2] = x[d+D/2] cos[d+D/2] + x[d] sin[d+D/2]  (fp32, one rounding).
// Consecutive threads walk (d-chunk, h, t, b) in that order, so reads are linear in x and every
// written row segment is 16 bytes x D/16 threads.
template <typename X>
__device__ __forceinline__ void load8(const X* p, float (&v)[8]) {
  if constexpr (sizeof(X) == 4) {
    const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  } else {
    const uint4 a = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) { const float2 f = Elem<X>::unpack(w[e]); v[2 * e] = f.x; v[2 * e + 1] = f.y; }
  }
}
__device__ __forceinline__ void load8_any(const void* p, size_t i, int dt, float (&v)[8]) {
  if (dt == NSA_FP32) load8(reinterpret_cast<const float*>(p) + i, v);
  else if (dt == NSA_FP16) load8(reinterpret_cast<const __half*>(p) + i, v);
  else load8(reinterpret_cast<const __nv_bfloat16*>(p) + i, v);
}

template <typename X, typename Y>
__global__ void __launch_bounds__(256) rope_to_heads_kernel(const X* __restrict__ x, Y* __restrict__ y,
                                                            const void* __restrict__ cosp, const void* __restrict__ sinp,
                                                            int B, int T, int H, int D, int cs_dt) {
  const int CH = D / 16;                                   // threads per row
  const long long total = (long long)B * T * H * CH;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int ch = (int)(i % CH);
    const long long row = i / CH;                          // (b, t, h)
    const int h = (int)(row % H);
    const long long bt = row / H;
    const int t = (int)(bt % T);
    const long long b = bt / T;
    const int d0 = ch * 8, d1 = D / 2 + ch * 8;
    float lo[8], hi[8];
    load8(x + (size_t)row * D + d0, lo);
    load8(x + (size_t)row * D + d1, hi);
    float olo[8], ohi[8];
    if (cosp != nullptr) {
      float c0[8], c1[8], s0[8], s1[8];
      load8_any(cosp, (size_t)t * D + d0, cs_dt, c0);
      load8_any(cosp, (size_t)t * D + d1, cs_dt, c1);
      load8_any(sinp, (size_t)t * D + d0, cs_dt, s0);
      load8_any(sinp, (size_t)t * D + d1, cs_dt, s1);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        olo[e] = fmaf(lo[e], c0[e], -hi[e] * s0[e]);
        ohi[e] = fmaf(hi[e], c1[e], lo[e] * s1[e]);
      }
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) { olo[e] = lo[e]; ohi[e] = hi[e]; }
    }
    Y* dst = y + (((size_t)b * H + h) * T + t) * D;
    *reinterpret_cast<uint4*>(dst + d0) = make_uint4(Elem<Y>::pack(olo[0], olo[1]), Elem<Y>::pack(olo[2], olo[3]),
                                                     Elem<Y>::pack(olo[4], olo[5]), Elem<Y>::pack(olo[6], olo[7]));
    *reinterpret_cast<uint4*>(dst + d1) = make_uint4(Elem<Y>::pack(ohi[0], ohi[1]), Elem<Y>::pack(ohi[2], ohi[3]),
                                                     Elem<Y>::pack(ohi[4], ohi[5]), Elem<Y>::pack(ohi[6], ohi[7]));
  }
}

int rope_to_heads(const void* x, void* y, const void* cosp, const void* sinp, int B, int T, int H, int D, int x_dt,
                  int cs_dt, int y_dt, cudaStream_t st) {
  const long long items = (long long)B * T * H * (D / 16);
  if (items == 0) return NSA_OK;
  const int grid = grid_for(items, 256);
#define NSA_ROPE(XT, YT) \
  rope_to_heads_kernel<XT, YT><<<grid, 256, 0, st>>>(reinterpret_cast<const XT*>(x), reinterpret_cast<YT*>(y), cosp, sinp, B, T, H, D, cs_dt)
  if (y_dt == NSA_BF16) {
    if (x_dt == NSA_FP32) NSA_ROPE(float, __nv_bfloat16);
    else if (x_dt == NSA_FP16) NSA_ROPE(__half, __nv_bfloat16);
    else NSA_ROPE(__nv_bfloat16, __nv_bfloat16);
  } else {
    if (x_dt == NSA_FP32) NSA_ROPE(float, __half);
    else if (x_dt == NSA_FP16) NSA_ROPE(__half, __half);
    else NSA_ROPE(__nv_bfloat16, __half);
  }
#undef NSA_ROPE
  return launch_status("rope_to_heads");
}

}  // namespace nsa
