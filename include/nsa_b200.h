/*
 * C ABI of the B200 (sm_100a) Native-Sparse-Attention kernels.
 *
 * Every entry point takes raw device pointers, sizes and a CUDA stream, launches
 * asynchronously on that stream, allocates nothing unless stated, and returns an
 * int status: NSA_OK (0) or a negative NSA_ERR_* code, with a description available
 * from nsa_last_error().  Tensors are dense row-major ("contiguous"):
 *   Q, out, dO, dQ   [B, H,   Tq, D]
 *   K, V, dK, dV     [B, Hkv, Tk, D]     H % Hkv == 0 (Hkv == H is the reference's case)
 *   lse, delta       [B, H,   Tq]  fp32
 *   block indices    [B, Hi,  nq, k] int32,  Hi == H (per query head) or Hkv (shared by a group)
 *   gate logits      [B, H,   Tq, 3]
 * Query rows align with the tail of the keys: key position of row i is i + (Tk - Tq).
 *
 * Each declaration cites the interface of the reference project
 * (qflen/nsa-from-scratch, paths relative to its root) that it stands in for.
 */
#ifndef NSA_B200_H
#define NSA_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* nsa_stream_t; /* a cudaStream_t; NULL is the default stream */

#define NSA_OK 0
#define NSA_ERR_ARG (-1)         /* a size, pointer or flag is out of range          */
#define NSA_ERR_UNSUPPORTED (-2) /* a combination no kernel is instantiated for      */
#define NSA_ERR_CUDA (-3)        /* the CUDA runtime reported an error               */
#define NSA_ERR_DEVICE (-4)      /* a kernel gave up on a bounded wait (status word) */

#define NSA_BF16 0
#define NSA_FP16 1
#define NSA_FP8_E4M3 2
#define NSA_FP8_E5M2 3
#define NSA_FP32 4

#define NSA_BRANCH_COMPRESSED 1
#define NSA_BRANCH_SELECTED 2
#define NSA_BRANCH_SLIDING 4

#define NSA_GATE_SIGMOID 0
#define NSA_GATE_SOFTMAX 1

/* Engine for nsa_attention_fwd: AUTO picks the tcgen05/TMA kernel when the shape
 * qualifies (bf16/fp16, D in {64,128}, 64-token blocks) and the generic
 * tensor-core kernel otherwise. */
#define NSA_ENGINE_AUTO 0
#define NSA_ENGINE_GENERIC 1
#define NSA_ENGINE_TCGEN05 2

const char* nsa_last_error(void);
int nsa_abi_version(void);

/* Mean over windows of `block` rows every `stride` rows:  x [B,H,T,D] -> out [B,H,n_out,D].
 * fp32 sum in row order, divide by `block`, one round-to-nearest-even to the output
 * type (16-bit inputs keep their type; fp8 inputs are first dequantised to
 * bf16(fp32(x)*dequant_scale) and produce bf16).  stride == block: n_out = ceil(T/block),
 * a trailing partial window is still divided by `block`.  stride < block: only whole
 * windows, n_out = (T-block)/stride + 1.
 * Replaces: _mean_pool, nsa/triton/compressed.py:25-44; the block means taken in
 * _resolve_block_indices, nsa/triton/forward.py:344-345. */
int nsa_pool_mean(const void* x, void* out, int B, int H, int T, int D, int block, int stride,
                  int n_out, int dtype, float dequant_scale, nsa_stream_t stream);

/* Learned pooling: out[b,h,c,:] = sum_s x[b,h,c*stride+s,:] * w[s,:] over the `block` rows of window c (rows past
 * the end count as zero, which is what the reference's zero padding gives); w [block, D] fp32, 16-byte aligned;
 * fp32 sum in row order, one rounding to the 16-bit type of x.  n_out as for nsa_pool_mean.
 * Replaces: torch.einsum("bhnsd,sd->bhnd", K_blocks, pool_proj_k), nsa/reference.py:109-113 (the reference's
 * kernels refuse pool="learned", nsa/triton/compressed.py:219-220; only its plain-torch path has it). */
int nsa_pool_learned(const void* x, const float* w, void* out, int B, int H, int T, int D, int block, int stride,
                     int n_out, int dtype, nsa_stream_t stream);

/* MoBA routing as a producer of block lists: every query TOKEN takes its top_k_per_query (<= 64) key blocks by
 * q . Kb[block] * scale (Kb [B,Hkv,nk,D]: key block means from nsa_pool_mean; block n legal for row i iff
 * !causal or n*bn <= i + offset, offset from the lengths padded to the block sizes); query block qb lists the union
 * of its bm rows' picks (rows past Tq count as zero rows, as in the padded tensor) in ascending order, padded with
 * the out-of-range id nk up to `cap` slots; a union larger than cap keeps the cap blocks with the best block-level
 * score (max over the rows), best first.  Ties resolve to the lowest block id; a row with fewer legal blocks than
 * picks contributes its legal ones only.  idx [B,H,nq,cap] int32, fed to the selected branch as block_indices.
 * Replaces: _per_query_top_k_indices, nsa/triton/moba.py:18-92. */
int nsa_moba_block_indices(const void* Q, const void* Kb, int32_t* idx, int B, int H, int Hkv, int Tq, int nq, int nk,
                           int D, int top_k_per_query, int cap, int bm, int bn, int offset, int causal, float scale,
                           int dtype, nsa_stream_t stream);

/* Block scoring + causal legality + top-k in one kernel.
 *   Qb [B,H,nq,D], Kb [B,Hkv,nk,D]: block means (nsa_pool_mean), 16-bit.
 *   idx [B,H,nq,k_out] int32, k_out = min(top_k, nk), ordered by descending score,
 *   ties (and the -inf slots of rows with fewer than k_out legal blocks) lowest index first.
 * score = fp32 dot over D (fma in index order) * scale; block c is legal for q block q iff
 * !causal or c*bn <= q*bm + bm-1 + offset.  force_first / force_local give score +inf to
 * the first blocks and to the last legal blocks of each row (0/0 = the reference).
 * shared_per_group != 0: one index row per KV head, idx [B,Hkv,nq,k_out]; its query vector is
 * the fp32 sum, in head order, of the block means of the H/Hkv query heads that share the KV
 * head (0 = the reference: one row per query head).
 * Replaces: _resolve_block_indices, nsa/triton/forward.py:321-359 (einsum + mask + topk). */
int nsa_select_blocks(const void* Qb, const void* Kb, int32_t* idx, int B, int H, int Hkv, int nq,
                      int nk, int D, int top_k, int bm, int bn, int offset, int causal, float scale,
                      int force_first, int force_local, int shared_per_group, int dtype,
                      nsa_stream_t stream);

/* Selection scores taken from the compressed branch's attention probabilities (the scorer of the NSA paper):
 *   scores[b,hi,qb,j] = sum over the rows i of query block qb (64 rows; and, shared_per_group != 0, over the
 *   H/Hkv query heads of KV head hi) of  sum_c exp(q_i . Kc_c * scale - lse[b,h,i]) * w(c,j),
 * lse [B,H,Tq] being the compressed branch's log-sum-exp (nsa_attention_fwd, branches = COMPRESSED, fused = 0)
 * and w(c,j) = |[c*stride, c*stride+block) intersect [j*bn, (j+1)*bn)| / block.  Compressed token c counts for
 * row i iff c*stride + block - 1 <= i + cmp_offset (or always, causal = 0).  Illegal selection blocks
 * (j*bn > qb*64 + 63 + sel_offset under causal) come out -inf, forced ones +inf; nsa_topk_from_scores then
 * gives the indices.  Sums are formed in a fixed order: results repeat bit for bit.
 * Replaces nothing in the reference, which scores with block means (nsa/triton/forward.py:321-359); the
 * scores enter its functions through their block_scores= / block_indices= arguments
 * (nsa/triton/selected.py:195-196). */
int nsa_cmp_block_scores(const void* Q, const void* Kc, const float* lse, float* scores, int B, int H, int Hkv,
                         int Tq, int Nc, int D, int nk, int cmp_block, int cmp_stride, int cmp_offset, int bn,
                         int sel_offset, int causal, float scale, int force_first, int force_local,
                         int shared_per_group, int dtype, nsa_stream_t stream);

/* The same scores on the tcgen05 tensor cores (D in {64,128}, 16-bit storage, 64-token selection blocks' score
 * rows must fit shared memory; NSA_ERR_UNSUPPORTED otherwise -- use nsa_cmp_block_scores then).  The product is
 * formed transposed (compressed tokens on the TMEM lanes), so the sum over query rows is a sum over one thread's
 * registers.  head_scratch: B*H*nq*nk floats the caller provides (per-head block sums before the group sum,
 * legality and forcing are applied); contents need not be preserved.  Sums are in a fixed order, but not the
 * order of nsa_cmp_block_scores: the two agree to fp32 rounding, not bit for bit. */
int nsa_cmp_block_scores_tc(const void* Q, const void* Kc, const float* lse, float* scores, float* head_scratch,
                            int B, int H, int Hkv, int Tq, int Nc, int D, int nk, int cmp_block, int cmp_stride,
                            int cmp_offset, int bn, int sel_offset, int causal, float scale, int force_first,
                            int force_local, int shared_per_group, int dtype, nsa_stream_t stream);

/* Top-k over caller-supplied fp32 scores [BH,nq,nk] with the same legality rule and order.
 * Replaces: _topk_indices_from_scores, nsa/triton/selected.py:153-185. */
int nsa_topk_from_scores(const float* scores, int32_t* idx, int BH, int nq, int nk, int top_k,
                         int bm, int bn, int offset, int causal, nsa_stream_t stream);

/* Arguments of the attention forward.  One launch evaluates the branches named in
 * `branches` for every 64-row query tile:
 *   fused == 0: exactly one branch; writes out (same 16-bit type as compute) and lse.
 *   fused == 1: writes out = sum_b gate_b * branch_b (gates from gate logits, or the
 *               constant of zero logits when gates == NULL); lse is not written.
 * Q (and K/V) may be fp8 with per-tensor scales; they are dequantised to bf16 as
 * bf16(fp32(x) * scale) while being staged.  kv_dtype is q_dtype, or NSA_BF16 beside an fp8 Q
 * (tcgen05 kernel only): K/V dequantised once by nsa_fp8_dequantize, so that a K/V tile is not
 * converted again by every query block that attends it; k_scale / v_scale are then unused. */
/* io_layout bits of nsa_fwd_args: the caller's token-major tensors used as they are
 * (nsa/model/llama_nsa.py:82 permutes the gate logits to [B,H,T,3] and :94 transposes the
 * result back to [B,T,H*D]; with these bits neither copy exists). */
#define NSA_IO_OUT_BTHD 1   /* out is [B,Tq,H,D] (= [B,Tq,H*D]) */
#define NSA_IO_GATES_BTHD 2 /* gates are [B,Tq,H,3] */

typedef struct nsa_fwd_args {
  const void* Q;       /* [B,H,Tq,D]   q_dtype                                    */
  const void* K;       /* [B,Hkv,Tk,D] kv_dtype                                   */
  const void* V;
  const void* Kc;      /* [B,Hkv,Nc,D] pooled keys/values, 16-bit (compressed)    */
  const void* Vc;
  const int32_t* idx;  /* [B,Hi,nq,top_k] (selected)                              */
  const void* gates;   /* [B,H,Tq,3] gate logits or NULL (fused)                  */
  void* out;           /* [B,H,Tq,D]                                              */
  float* lse;          /* [B,H,Tq] or NULL                                        */
  int32_t B, H, Hkv, Hi;
  int32_t Tq, Tk, D;
  int32_t offset;                                /* key position of query row i is i + offset (normally Tk-Tq) */
  int32_t Nc, cmp_block, cmp_stride, cmp_offset; /* pooled token c visible iff c*stride+block-1 <= i+cmp_offset */
  int32_t nq, top_k, bm, bn, sel_key_limit;      /* keys j < sel_key_limit attendable (padded Tk)           */
  int32_t window;
  int32_t causal;
  int32_t branches, fused, gate_act;
  int32_t q_dtype, kv_dtype, gate_dtype;         /* NSA_* dtype codes; out has the compute type             */
  float scale;                                   /* softmax scale                                          */
  float q_scale, k_scale, v_scale;               /* fp8 dequantisation scales                              */
  int32_t engine;                                /* NSA_ENGINE_*                                           */
  int32_t io_layout;                             /* NSA_IO_* bits; 0 = every tensor [B,H,T,.]              */
  /* Decoding-sized launches (few query blocks, long key ranges): nsplit > 1 (at most 16) spreads each work item's key
   * tiles over nsplit thread blocks and merges their partial results in a second kernel.  Fused launches on
   * the tcgen05 kernel with 16-bit storage only (ignored elsewhere).  The caller supplies the scratch:
   * B*H*Tq*nsplit*3*(D+4)*4 bytes, 16-byte aligned; its contents need not be preserved or cleared. */
  int32_t nsplit;
  void* split_scratch;
  int64_t split_scratch_bytes;
  /* Optional: the number of filled key positions, read from device memory when the kernel starts.  With it
   * K/V (and Kc/Vc) are allocations longer than what is filled, Tk / Nc give the allocated lengths, and
   * offset, cmp_offset and sel_key_limit are derived on the device from *dyn_len -- so the launch can sit in a
   * CUDA graph that is replayed while a KV cache grows.  Needs causal = 1, fused = 1, 16-bit storage, the
   * tcgen05 kernel and the split scratch (nsplit >= 1); NSA_ERR_UNSUPPORTED otherwise. */
  const int32_t* dyn_len;
  /* Fused launches only.  accumulate != 0: `out` already holds a gated partial sum (an earlier fused launch with
   * other branches) and this launch adds its branches to it -- the three branches may thus be spread over several
   * launches, e.g. the compressed branch first when the selection is scored from its probabilities.  tcgen05 kernel
   * only.  A fused launch of exactly ONE branch may also return that branch's lse (lse != NULL). */
  int32_t accumulate;
} nsa_fwd_args;

/* Replaces the kernels behind compressed_attention (nsa/triton/compressed.py:191-300),
 * selected_attention (nsa/triton/selected.py:188-315), sliding_attention
 * (nsa/triton/sliding.py:136-205), the dequantise-then-attend of selected_attention_fp8
 * (nsa/triton/fp8.py:43-75) and, with fused=1, the branch launches plus combine of
 * nsa_forward (nsa/triton/forward.py:362-406). */
int nsa_attention_fwd(const nsa_fwd_args* args, nsa_stream_t stream);

/* Synchronises `stream`, then reports whether any kernel launched so far gave up on one of
 * its bounded device-side waits: NSA_OK, or NSA_ERR_DEVICE (and the condition is cleared).
 * No counterpart in the reference (its kernels have no device-side waits). */
int nsa_device_status(nsa_stream_t stream);

/* Test hook: writes `value` into the device status word of a kernel family (0 = attention forward,
 * 2 = attention backward) from the host, as a kernel does when one of its bounded waits expires; the
 * next nsa_device_status() must then report NSA_ERR_DEVICE and clear it.  Lets the error path be
 * exercised without making any kernel wait.  No counterpart in the reference. */
int nsa_debug_set_device_status(int kernel_family, int value);

/* Compressed-branch forward that needs no scratch memory from the caller: the pooled K and V
 * live in an array built into the library (NSA_STATIC_SCRATCH_BYTES per GPU, held until the
 * process exits).  Meant for hosts that cannot allocate at call time -- a runtime whose device
 * memory is fully planned up front, or code inside a region where cudaMalloc is forbidden or
 * would stall the device.  Same results as nsa_pool_mean (K, V) followed by
 * nsa_attention_fwd(branches = NSA_BRANCH_COMPRESSED, fused = 0): out [B,H,Tq,D], lse [B,H,Tq]
 * (lse may be NULL).  Limit: B*Hkv*n_pooled*D*4 bytes (each half rounded up to 256) must fit the
 * array, otherwise NSA_ERR_UNSUPPORTED with the sizes in nsa_last_error().  The first call on a
 * device looks up the array's device address (cudaGetSymbolAddress); make that first call
 * outside any stream capture.  All calls share the one array: calls that may run concurrently
 * on the GPU race with each other; nothing in it needs clearing between calls.
 * No counterpart in the reference (its wrappers allocate through torch). */
#define NSA_STATIC_SCRATCH_BYTES (16u << 20)
int nsa_compressed_attention_static(const void* Q, const void* K, const void* V, void* out, float* lse, int B,
                                    int H, int Hkv, int Tq, int Tk, int D, int block, int stride, int causal,
                                    float scale, int dtype, nsa_stream_t stream);

/* The reference's native launcher, same argument list (bf16, Hkv == H folded into BH,
 * 64x64 blocks, pre-padded lengths, D in {32,64,128}); returns a status instead of void.
 * Replaces: launch_selected_attn_fwd, nsa/cuda/selected_fwd.cu:582-614
 * (declared at nsa/cuda/bindings.cpp:14-20). */
int launch_selected_attn_fwd(const void* Q, const void* K, const void* V, const int* Idx, void* Out,
                             float* Lse, int BH, int n_q_blocks, int Tq_p, int Tk_p, int D, int top_k,
                             int offset, int causal, float sm_scale, nsa_stream_t stream);

/* delta[r] = sum_d dO[r,d] * O[r,d] in fp32 for `rows` rows of D 16-bit elements.
 * Replaces: D_vec = (dO.float()*O.float()).sum(-1), nsa/triton/backward.py:158. */
int nsa_bwd_delta(const void* dO, const void* O, float* delta, int64_t rows, int D, int dtype,
                  nsa_stream_t stream);

/* Attention backward of ONE branch (nsa_bwd_args.branch = NSA_BRANCH_SELECTED / _SLIDING /
 * _COMPRESSED).  dQ [B,H,Tq,D] is WRITTEN (each query tile is owned by one
 * thread block) in dq_dtype (NSA_FP32 or the 16-bit input type).  dK_f, dV_f
 * [B,Hkv,Tk,D] are fp32 and are ACCUMULATED into (the caller zeroes them); the sum over the
 * query heads that share a KV head is formed here too.  Rows with lse = -inf contribute nothing.
 *
 * Two engines.  The tcgen05 engine (selected branch, 16-bit storage, D in {64,128}, 64x64 blocks,
 * top_k <= 256) uses no floating-point atomics: it inverts the block lists (per key block, the
 * query blocks that chose it), accumulates dK/dV of a key block in tensor memory over that
 * list and writes them once, and forms dQ in a second, query-major pass; every sum has a fixed
 * order, so dQ, dK and dV repeat bit for bit.  It needs caller-supplied scratch of
 * nsa_attention_bwd_scratch_bytes() bytes (256-byte aligned; contents need neither be cleared nor
 * preserved).  The generic engine (every other shape and branch; mma.sync) adds its dK/dV tiles
 * with fp32 atomic adds, so their last bits depend on the order of arrival.
 * engine = NSA_ENGINE_AUTO takes tcgen05 when the shape qualifies AND scratch is given, else generic;
 * NSA_ENGINE_TCGEN05 fails with NSA_ERR_UNSUPPORTED / NSA_ERR_ARG instead of falling back. */
typedef struct nsa_bwd_args {
  const void* Q;
  const void* K;
  const void* V;
  const void* dO;
  const float* lse;
  const float* delta;
  const int32_t* idx;
  void* dQ;
  float* dK_f;
  float* dV_f;
  int32_t B, H, Hkv, Hi;
  int32_t Tq, Tk, D;
  int32_t nq, top_k, bm, bn, sel_key_limit;
  int32_t offset; /* key position of row i is i + offset */
  int32_t causal;
  int32_t dtype, dq_dtype;
  float scale;
  int32_t branch;                               /* NSA_BRANCH_*; 0 is taken as NSA_BRANCH_SELECTED            */
  int32_t window;                               /* sliding                                                     */
  int32_t Nc, cmp_block, cmp_stride, cmp_offset; /* compressed: K, V, dK_f, dV_f are then [B,Hkv,Nc,D] (pooled) */
  int32_t engine;                                /* NSA_ENGINE_*                                                */
  void* scratch;                                 /* tcgen05 engine: nsa_attention_bwd_scratch_bytes() bytes      */
  int64_t scratch_bytes;
} nsa_bwd_args;

/* Bytes of scratch the tcgen05 engine needs for this problem (0 when the shape does not qualify, so that
 * the generic engine will run; negative NSA_ERR_* on a NULL argument).  Holds the inverted block lists, the
 * work items and the partial dK/dV sums of key blocks whose list is split over several thread blocks.
 * No counterpart in the reference (its kernel adds every tile atomically, nsa/triton/backward.py:98-118). */
int64_t nsa_attention_bwd_scratch_bytes(const nsa_bwd_args* args);

/* Replaces: selected_backward / _bwd_kernel, nsa/triton/backward.py:16-195 (branch forced to selected). */
int nsa_selected_bwd(const nsa_bwd_args* args, nsa_stream_t stream);

/* Any branch.  lse and delta are those of the branch's own forward output.  Replaces the
 * autograd-through-reference backward of the compressed and sliding branches,
 * nsa/triton/forward.py:133-140 and :273-298. */
int nsa_attention_bwd(const nsa_bwd_args* args, nsa_stream_t stream);

/* Backward of nsa_pool_mean for fp32 gradients: dx [B,H,T,D] += spread(dxc [B,H,n_out,D]) / block,
 * every row receiving the gradients of the windows that cover it.
 * Replaces: the autograd of view(...).mean(3), nsa/reference.py:102-108. */
int nsa_pool_mean_bwd(const float* dxc, float* dx, int B, int H, int T, int D, int block, int stride, int n_out,
                      nsa_stream_t stream);

/* The reference's native backward launcher, same argument list: dQ is bf16 and is
 * written; dK_f/dV_f are fp32 and accumulated into (zeroed by the caller, as
 * nsa/cuda/bindings.cpp:160-162 does).  Returns a status instead of void.  The argument list has
 * no room for scratch, so at D in {64,128} this entry point takes the tcgen05 engine's scratch
 * from the stream-ordered allocator (cudaMallocAsync / cudaFreeAsync on `stream`): the one
 * place in this library that allocates.
 * Replaces: launch_selected_attn_bwd, nsa/cuda/selected_bwd.cu:731-772
 * (declared at nsa/cuda/bindings.cpp:22-30). */
int launch_selected_attn_bwd(const void* Q, const void* K, const void* V, const void* dO,
                             const float* LSE, const float* Dvec, const int* Idx, void* dQ, float* dK_f,
                             float* dV_f, int BH, int n_q_blocks, int Tq_p, int Tk_p, int D, int top_k,
                             int offset, int causal, float sm_scale, nsa_stream_t stream);

/* out = g0*out_c + g1*out_s + g2*out_w per row, g = sigmoid or softmax of the logits.
 * With 16-bit gates the gate, each product and each sum are rounded to the 16-bit type
 * in that order (what the reference's tensor expression does); with fp32 gates the
 * result is fp32.  rows = B*H*Tq.
 * Replaces: combine, nsa/triton/gating.py:15-40. */
int nsa_combine(const void* out_c, const void* out_s, const void* out_w, const void* gates, void* out,
                int64_t rows, int D, int activation, int dtype, int gate_dtype, nsa_stream_t stream);

/* absmax[0] = max(|x|) over n elements (fp32 result; the caller zeroes absmax first).
 * Replaces: x.abs().max(), nsa/triton/fp8.py:37. */
int nsa_fp8_absmax(const void* x, int64_t n, int dtype, float* absmax, nsa_stream_t stream);

/* out8[i] = saturating_cast_fp8( round_to_dtype(x[i] / scale) ).
 * Replaces: (x/scale).clamp(-max,max).to(fmt), nsa/triton/fp8.py:39-40. */
int nsa_fp8_quantize(const void* x, void* out8, int64_t n, int dtype, int fmt, float scale,
                     nsa_stream_t stream);

/* out[i] = bf16( fp32(x8[i]) * scale ), n elements; x8 holds `fmt` (NSA_FP8_E4M3 / NSA_FP8_E5M2) bytes, both
 * pointers 16-byte aligned.  The operands the reference's wrapper builds before it attends; with GQA, K and V
 * are a small fraction of Q, so the forward dequantises them once here and converts only Q inside the kernel.
 * Replaces: Q.to(torch.bfloat16) * scale_q etc., nsa/triton/fp8.py:67-69. */
int nsa_fp8_dequantize(const void* x8, void* out, int64_t n, int fmt, float scale, nsa_stream_t stream);

/* dst (16-bit `dtype`) = round(src fp32), n elements.
 * Replaces: dQ_f.to(Q.dtype) etc., nsa/triton/backward.py:195. */
int nsa_cast_from_f32(const float* src, void* dst, int64_t n, int dtype, nsa_stream_t stream);

/* y[b,h,t,:] = rope(x[b,t,h,:]) rounded once to `y_dtype` (bf16/fp16): the head-major, 16-bit,
 * position-encoded tensor the attention kernels read, made from the projection output
 * x [B,T,H,D] (`x_dtype` fp32, bf16 or fp16) in one pass.  rope(x)[d] = x[d]*cos[t,d] +
 * rot(x)[d]*sin[t,d] with rot(x) = (-x[D/2:], x[:D/2]) in fp32; cos/sin [T,D] in `cs_dtype`; with
 * cos == NULL the values are only transposed and cast (the V path).
 * Replaces: .view(B,T,H,D).transpose(1,2), _apply_rope and .to(bf16) of the caller,
 * nsa/model/llama_nsa.py:77-80,91 and nsa/model/llama_dense.py:19-37. */
int nsa_rope_to_heads(const void* x, void* y, const void* cos, const void* sin, int B, int T, int H, int D,
                      int x_dtype, int cs_dtype, int y_dtype, nsa_stream_t stream);

/* KV-cache append, one launch: k_new, v_new [B,Hkv,t_new,D] become rows filled..filled+t_new-1 of K, V
 * [B,Hkv,max_len,D]; the pooled windows (cmp_block / cmp_stride, nsa_pool_mean's rules) of Kc, Vc
 * [B,Hkv,nc_alloc,D] and the selection-block means Kb [B,Hkv,nb_alloc,D] that contain a new row are recomputed
 * with nsa_pool_mean's arithmetic.  Afterwards Kc/Vc/Kb hold what nsa_pool_mean gives on the filled prefix.
 * No counterpart in the reference (it recomputes the pooled tensors from scratch in every call,
 * nsa/triton/compressed.py:25-44, nsa/triton/forward.py:344-345). */
int nsa_cache_append(const void* k_new, const void* v_new, void* K, void* V, void* Kc, void* Vc, void* Kb, int B,
                     int Hkv, int D, int t_new, int filled, int max_len, int nc_alloc, int nb_alloc, int cmp_block,
                     int cmp_stride, int sel_block, int dtype, nsa_stream_t stream);

/* The two launches above for a cache whose fill count lives in DEVICE memory, so that a decoding step can be
 * captured into a CUDA graph once and replayed while the cache grows.
 * nsa_cache_append_dev: appends at *filled, then adds t_new to *filled (a second, one-thread launch); an
 *   append that would pass max_len writes nothing and leaves *filled alone (the host, which mirrors the
 *   count, should refuse it first).
 * nsa_select_blocks_cached: nsa_select_blocks with causal = 1 and the block-grid offset derived from
 *   *filled (ceil(filled/bn)*bn - nq*bm); Kb [B,Hkv,nk_alloc,D] is the cache's whole block-mean tensor.
 * No counterpart in the reference. */
int nsa_cache_append_dev(const void* k_new, const void* v_new, void* K, void* V, void* Kc, void* Vc, void* Kb,
                         int B, int Hkv, int D, int t_new, int32_t* filled, int max_len, int nc_alloc, int nb_alloc,
                         int cmp_block, int cmp_stride, int sel_block, int dtype, nsa_stream_t stream);
int nsa_select_blocks_cached(const void* Qb, const void* Kb, int32_t* idx, int B, int H, int Hkv, int nq,
                             int nk_alloc, int D, int top_k, int bm, int bn, const int32_t* filled, float scale,
                             int force_first, int force_local, int shared_per_group, int dtype,
                             nsa_stream_t stream);

/* Strided copy between host and device on `stream`: `rows` rows of `row_bytes` bytes, row r at
 * dst + r*dst_pitch / src + r*src_pitch; to_device = 1 host->device, 0 device->host.  Asynchronous when
 * the host side is pinned.  Lets the host-tensor entry point move the [heads, chunk, D] slab of one
 * (batch, KV head, query chunk) unit in a single call.
 * Replaces: the .to(device) / .cpu() copies a caller of nsa_forward does around it
 * (nsa/bench/throughput.py:78-80 creates its inputs with torch.randn(..., device=device)). */
int nsa_memcpy_2d(void* dst, size_t dst_pitch, const void* src, size_t src_pitch, size_t row_bytes,
                  size_t rows, int to_device, nsa_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* NSA_B200_H */
