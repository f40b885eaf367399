// Compressed-branch forward for callers that cannot hand this library any scratch memory.
//
// Who that is: a host runtime that carved up all of its device memory before start-up and runs
// with the allocator switched off (an inference server with a fixed memory plan), or code that
// sits inside a region where cudaMalloc is illegal or unwanted because it can stall the whole
// device (stream capture, a latency-critical decode loop).  The normal path needs two pooled
// tensors (mean-pooled K and V) that somebody must allocate; here they live in a fixed array that
// is part of the library image, so the call needs nothing but its inputs and outputs.
//
// The price: the array is NSA_STATIC_SCRATCH_BYTES large on every GPU that loads the library, for
// the life of the process; problems whose pooled K/V do not fit are refused; and every call uses
// the same array, so two calls that can overlap on the GPU (different streams, no dependency)
// corrupt each other.  Nothing in the array has to start at zero: each call overwrites all
// pooled rows it later reads, so stale contents of an earlier call are harmless.
#include "common.cuh"

#include <atomic>

namespace nsa {

int pool_mean(const void*, void*, int, int, int, int, int, int, int, int, float, cudaStream_t);

static __device__ __align__(256) unsigned char g_static_scratch[NSA_STATIC_SCRATCH_BYTES];

// Device address of the array on the current device.  In host code the symbol's name is only a
// handle, not a pointer a kernel could use; the address comes from cudaGetSymbolAddress, asked
// once per device with that device current.
static int scratch_address(unsigned char** out, cudaStream_t st) {
  constexpr int kMaxDevices = 64;
  static std::atomic<unsigned char*> cached[kMaxDevices];   // zero-initialised; racing first calls store the same address
  int dev = -1;
  NSA_CUDA_OK(cudaGetDevice(&dev));
  NSA_REQUIRE(dev >= 0 && dev < kMaxDevices, NSA_ERR_UNSUPPORTED, "static scratch: device index %d out of range", dev);
  unsigned char* p = cached[dev].load(std::memory_order_acquire);
  if (p == nullptr) {
    // the look-up is not a stream operation: made while `st` is being captured it could invalidate the capture
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    NSA_CUDA_OK(cudaStreamIsCapturing(st, &cap));
    NSA_REQUIRE(cap == cudaStreamCaptureStatusNone, NSA_ERR_UNSUPPORTED,
                "static scratch: the first call on a device looks up the array's address and must come before any stream capture");
    void* q = nullptr;
    NSA_CUDA_OK(cudaGetSymbolAddress(&q, g_static_scratch));
    NSA_REQUIRE(q != nullptr, NSA_ERR_CUDA, "static scratch: cudaGetSymbolAddress returned NULL");
    p = static_cast<unsigned char*>(q);
    cached[dev].store(p, std::memory_order_release);
  }
  *out = p;
  return NSA_OK;
}

}  // namespace nsa

using namespace nsa;

extern "C" int nsa_compressed_attention_static(const void* Q, const void* K, const void* V, void* out, float* lse, int B,
                                               int H, int Hkv, int Tq, int Tk, int D, int block, int stride, int causal,
                                               float scale, int dtype, nsa_stream_t stream) {
  NSA_REQUIRE(Q && K && V && out, NSA_ERR_ARG, "compressed (static scratch): NULL pointer");
  NSA_REQUIRE(dtype == NSA_BF16 || dtype == NSA_FP16, NSA_ERR_UNSUPPORTED, "compressed (static scratch): dtype %d", dtype);
  NSA_REQUIRE(B > 0 && Hkv > 0 && H > 0 && Tq > 0 && Tk > 0 && D > 0, NSA_ERR_ARG, "compressed (static scratch): empty problem");
  NSA_REQUIRE(block > 0 && stride > 0 && stride <= block, NSA_ERR_ARG, "compressed (static scratch): block %d stride %d", block, stride);
  const long long n_out = stride == block ? (Tk + block - 1) / block : (Tk >= block ? (Tk - block) / stride + 1 : 0);
  const long long one = ((long long)B * Hkv * n_out * D * 2 + 255) / 256 * 256;      // pooled K (or V), 256-byte aligned
  NSA_REQUIRE(2 * one <= (long long)NSA_STATIC_SCRATCH_BYTES, NSA_ERR_UNSUPPORTED,
              "compressed (static scratch): pooled K and V need %lld bytes, the built-in scratch holds %u "
              "(B*Hkv*n_pooled*D*4 must not exceed it); use nsa_pool_mean + nsa_attention_fwd with your own buffers",
              2 * one, (unsigned)NSA_STATIC_SCRATCH_BYTES);
  unsigned char* base = nullptr;
  cudaStream_t st = (cudaStream_t)stream;
  int rc = scratch_address(&base, st);
  if (rc != NSA_OK) return rc;
  void* Kc = base;
  void* Vc = base + one;
  if ((rc = pool_mean(K, Kc, B, Hkv, Tk, D, block, stride, (int)n_out, dtype, 1.f, st)) != NSA_OK) return rc;
  if ((rc = pool_mean(V, Vc, B, Hkv, Tk, D, block, stride, (int)n_out, dtype, 1.f, st)) != NSA_OK) return rc;
  nsa_fwd_args a = {};
  a.Q = Q; a.K = K; a.V = V; a.Kc = Kc; a.Vc = Vc; a.out = out; a.lse = lse;
  a.B = B; a.H = H; a.Hkv = Hkv; a.Hi = H; a.Tq = Tq; a.Tk = Tk; a.D = D; a.offset = Tk - Tq;
  a.Nc = (int)n_out; a.cmp_block = block; a.cmp_stride = stride;
  a.cmp_offset = (stride == block ? (int)n_out * block : Tk) - Tq;
  a.causal = causal; a.branches = NSA_BRANCH_COMPRESSED; a.fused = 0;
  a.q_dtype = a.kv_dtype = dtype; a.scale = scale; a.engine = NSA_ENGINE_AUTO;
  return nsa_attention_fwd(&a, stream);
}
