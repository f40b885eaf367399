// extern "C" boundary: argument validation, error text, dispatch to the kernels.
#include "common.cuh"

#include <stdarg.h>
#include <stdio.h>

namespace nsa {

static thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

// kernels (other translation units)
int pool_mean(const void*, void*, int, int, int, int, int, int, int, int, float, cudaStream_t);
int moba_route(const void*, const void*, int32_t*, int, int, int, int, int, int, int, int, int, int, int, int, int, float, int, cudaStream_t);
int pool_weighted(const void*, const float*, void*, int, int, int, int, int, int, int, int, cudaStream_t);
int select_blocks(const void*, const void*, int32_t*, int, int, int, int, int, int, int, int, int, int, int, float, int,
                  int, int, int, const int32_t*, cudaStream_t);
int topk_from_scores(const float*, int32_t*, int, int, int, int, int, int, int, int, cudaStream_t);
int attention_fwd_generic(const nsa_fwd_args&, cudaStream_t);
int attention_fwd_tc5(const nsa_fwd_args&, cudaStream_t);
bool attention_fwd_tc5_supports(const nsa_fwd_args&);
int tc5_take_status(cudaStream_t, int*);
int attention_bwd(const nsa_bwd_args&, cudaStream_t);
bool attention_bwd_tc5_supports(const nsa_bwd_args&);
long long attention_bwd_tc5_scratch_bytes(const nsa_bwd_args&);
int attention_bwd_tc5(const nsa_bwd_args&, void*, long long, cudaStream_t);
int bw5_take_status(int*);
int tc5_set_status(int);
int bw5_set_status(int);
int pool_mean_bwd(const float*, float*, int, int, int, int, int, int, int, cudaStream_t);
int combine(const void*, const void*, const void*, const void*, void*, long long, int, int, int, int, cudaStream_t);
int fp8_absmax(const void*, long long, int, float*, cudaStream_t);
int fp8_quantize(const void*, void*, long long, int, int, float, cudaStream_t);
int fp8_dequantize(const void*, void*, long long, int, float, cudaStream_t);
int bwd_delta(const void*, const void*, float*, long long, int, int, cudaStream_t);
int cast_from_f32(const float*, void*, long long, int, cudaStream_t);
int cache_append(const void*, const void*, void*, void*, void*, void*, void*, int, int, int, int, int, int32_t*, int, int, int, int, int,
                 int, int, cudaStream_t);
int cmp_block_scores(const void*, const void*, const float*, float*, int, int, int, int, int, int, int, int, int, int, int, int, int, float,
                     int, int, int, int, cudaStream_t);
bool cmp_scores_tc5_supports(int, int, int, int, int, int);
int cmp_block_scores_tc5(const void*, const void*, const float*, float*, float*, int, int, int, int, int, int, int, int, int, int, int, int,
                         int, float, int, int, int, int, cudaStream_t);
int cs5_take_status(int*);
int rope_to_heads(const void*, void*, const void*, const void*, int, int, int, int, int, int, int, cudaStream_t);

static bool is16(int dt) { return dt == NSA_BF16 || dt == NSA_FP16; }
static bool is8(int dt) { return dt == NSA_FP8_E4M3 || dt == NSA_FP8_E5M2; }

static int check_fwd(const nsa_fwd_args& a) {
  NSA_REQUIRE(a.Q && a.out, NSA_ERR_ARG, "attention forward: Q/out pointer is NULL");
  NSA_REQUIRE(a.B > 0 && a.H > 0 && a.Hkv > 0 && a.H % a.Hkv == 0, NSA_ERR_ARG,
              "attention forward: B=%d H=%d Hkv=%d (H must be a multiple of Hkv)", a.B, a.H, a.Hkv);
  NSA_REQUIRE(a.Tq > 0 && a.Tk > 0, NSA_ERR_ARG, "attention forward: Tq=%d Tk=%d", a.Tq, a.Tk);
  NSA_REQUIRE(a.D == 32 || a.D == 64 || a.D == 128, NSA_ERR_UNSUPPORTED, "attention forward: head dim %d not in {32,64,128}", a.D);
  NSA_REQUIRE(is16(a.q_dtype) || is8(a.q_dtype), NSA_ERR_UNSUPPORTED, "attention forward: q dtype %d", a.q_dtype);
  NSA_REQUIRE(a.kv_dtype == a.q_dtype || (is8(a.q_dtype) && a.kv_dtype == NSA_BF16), NSA_ERR_UNSUPPORTED,
              "attention forward: K/V dtype %d with Q dtype %d (K/V share Q's type, or are bf16 beside an fp8 Q)", a.kv_dtype, a.q_dtype);
  const int br = a.branches;
  NSA_REQUIRE(br > 0 && br < 8, NSA_ERR_ARG, "attention forward: branch mask %d", br);
  NSA_REQUIRE(a.nsplit >= 0 && a.nsplit <= 16, NSA_ERR_ARG, "attention forward: nsplit %d not in [0, 16]", a.nsplit);
  NSA_REQUIRE((a.io_layout & ~(NSA_IO_OUT_BTHD | NSA_IO_GATES_BTHD)) == 0, NSA_ERR_ARG, "attention forward: io_layout %d has unknown bits", a.io_layout);
  if (!a.fused) {
    NSA_REQUIRE(br == 1 || br == 2 || br == 4, NSA_ERR_ARG, "attention forward: unfused launch needs exactly one branch (mask %d)", br);
  } else {
    NSA_REQUIRE(a.gate_act == NSA_GATE_SIGMOID || a.gate_act == NSA_GATE_SOFTMAX, NSA_ERR_ARG, "attention forward: gate activation %d", a.gate_act);
    NSA_REQUIRE(!a.gates || is16(a.gate_dtype) || a.gate_dtype == NSA_FP32, NSA_ERR_UNSUPPORTED, "attention forward: gate dtype %d", a.gate_dtype);
    NSA_REQUIRE(a.lse == nullptr || br == 1 || br == 2 || br == 4, NSA_ERR_ARG,
                "attention forward: a fused launch returns an lse only for a single branch (mask %d)", br);
  }
  NSA_REQUIRE(a.accumulate == 0 || (a.fused && a.nsplit <= 1 && a.dyn_len == nullptr), NSA_ERR_ARG,
              "attention forward: accumulate needs a fused, unsplit launch");
  if (br & NSA_BRANCH_COMPRESSED) {
    NSA_REQUIRE(a.Nc >= 0 && (a.Nc == 0 || (a.Kc && a.Vc)), NSA_ERR_ARG, "compressed: pooled K/V pointer is NULL");
    NSA_REQUIRE(a.cmp_block > 0 && a.cmp_stride > 0 && a.cmp_stride <= a.cmp_block, NSA_ERR_ARG,
                "compressed: block %d stride %d", a.cmp_block, a.cmp_stride);
  }
  if (br & (NSA_BRANCH_SELECTED | NSA_BRANCH_SLIDING)) NSA_REQUIRE(a.K && a.V, NSA_ERR_ARG, "attention forward: K/V pointer is NULL");
  if (br & NSA_BRANCH_SELECTED) {
    NSA_REQUIRE(a.idx, NSA_ERR_ARG, "selected: block index pointer is NULL");
    NSA_REQUIRE(a.bm > 0 && a.bn > 0 && a.top_k > 0, NSA_ERR_ARG, "selected: bm=%d bn=%d top_k=%d", a.bm, a.bn, a.top_k);
    NSA_REQUIRE(a.Hi == a.H || a.Hi == a.Hkv, NSA_ERR_ARG, "selected: index heads %d is neither H nor Hkv", a.Hi);
    NSA_REQUIRE(a.nq == (a.Tq + a.bm - 1) / a.bm, NSA_ERR_ARG, "selected: nq %d != ceil(Tq/bm)", a.nq);
    NSA_REQUIRE(a.sel_key_limit >= a.Tk && a.sel_key_limit < a.Tk + a.bn, NSA_ERR_ARG,
                "selected: key limit %d must be Tk padded to the block size", a.sel_key_limit);
  }
  if (br & NSA_BRANCH_SLIDING) NSA_REQUIRE(a.window >= 1, NSA_ERR_ARG, "sliding: window %d", a.window);
  return NSA_OK;
}

}  // namespace nsa

using namespace nsa;

extern "C" {

const char* nsa_last_error(void) { return g_err; }
int nsa_abi_version(void) { return 7; }

int nsa_pool_mean(const void* x, void* out, int B, int H, int T, int D, int block, int stride, int n_out, int dtype,
                  float dequant_scale, nsa_stream_t stream) {
  NSA_REQUIRE(x && out, NSA_ERR_ARG, "pool: NULL pointer");
  return pool_mean(x, out, B, H, T, D, block, stride, n_out, dtype, dequant_scale, (cudaStream_t)stream);
}

int nsa_pool_learned(const void* x, const float* w, void* out, int B, int H, int T, int D, int block, int stride, int n_out,
                     int dtype, nsa_stream_t stream) {
  NSA_REQUIRE(x && w && out, NSA_ERR_ARG, "pool (learned): NULL pointer");
  return pool_weighted(x, w, out, B, H, T, D, block, stride, n_out, dtype, (cudaStream_t)stream);
}

int nsa_moba_block_indices(const void* Q, const void* Kb, int32_t* idx, int B, int H, int Hkv, int Tq, int nq, int nk, int D,
                           int top_k_per_query, int cap, int bm, int bn, int offset, int causal, float scale, int dtype,
                           nsa_stream_t stream) {
  NSA_REQUIRE(Q && Kb && idx, NSA_ERR_ARG, "moba routing: NULL pointer");
  return moba_route(Q, Kb, idx, B, H, Hkv, Tq, nq, nk, D, top_k_per_query, cap, bm, bn, offset, causal, scale, dtype,
                    (cudaStream_t)stream);
}

int nsa_select_blocks(const void* Qb, const void* Kb, int32_t* idx, int B, int H, int Hkv, int nq, int nk, int D,
                      int top_k, int bm, int bn, int offset, int causal, float scale, int force_first, int force_local,
                      int shared_per_group, int dtype, nsa_stream_t stream) {
  NSA_REQUIRE(Qb && Kb && idx, NSA_ERR_ARG, "select: NULL pointer");
  return select_blocks(Qb, Kb, idx, B, H, Hkv, nq, nk, D, top_k, bm, bn, offset, causal, scale, force_first,
                       force_local, shared_per_group, dtype, nullptr, (cudaStream_t)stream);
}

int nsa_select_blocks_cached(const void* Qb, const void* Kb, int32_t* idx, int B, int H, int Hkv, int nq, int nk_alloc, int D,
                             int top_k, int bm, int bn, const int32_t* filled, float scale, int force_first, int force_local,
                             int shared_per_group, int dtype, nsa_stream_t stream) {
  NSA_REQUIRE(Qb && Kb && idx && filled, NSA_ERR_ARG, "select (cached): NULL pointer");
  return select_blocks(Qb, Kb, idx, B, H, Hkv, nq, nk_alloc, D, top_k, bm, bn, 0, 1, scale, force_first, force_local,
                       shared_per_group, dtype, filled, (cudaStream_t)stream);
}

int nsa_cmp_block_scores(const void* Q, const void* Kc, const float* lse, float* scores, int B, int H, int Hkv, int Tq, int Nc,
                         int D, int nk, int cmp_block, int cmp_stride, int cmp_offset, int bn, int sel_offset, int causal,
                         float scale, int force_first, int force_local, int shared_per_group, int dtype, nsa_stream_t stream) {
  NSA_REQUIRE(Q && Kc && lse && scores, NSA_ERR_ARG, "compressed scores: NULL pointer");
  NSA_REQUIRE(force_first >= 0 && force_local >= 0, NSA_ERR_ARG, "compressed scores: negative forced-block counts");
  return cmp_block_scores(Q, Kc, lse, scores, B, H, Hkv, Tq, Nc, D, nk, cmp_block, cmp_stride, cmp_offset, bn, sel_offset, causal,
                          scale, force_first, force_local, shared_per_group, dtype, (cudaStream_t)stream);
}

int nsa_cmp_block_scores_tc(const void* Q, const void* Kc, const float* lse, float* scores, float* head_scratch, int B, int H, int Hkv,
                            int Tq, int Nc, int D, int nk, int cmp_block, int cmp_stride, int cmp_offset, int bn, int sel_offset,
                            int causal, float scale, int force_first, int force_local, int shared_per_group, int dtype,
                            nsa_stream_t stream) {
  NSA_REQUIRE(Q && Kc && lse && scores && head_scratch, NSA_ERR_ARG, "compressed scores: NULL pointer");
  NSA_REQUIRE(B > 0 && H > 0 && Hkv > 0 && H % Hkv == 0 && Tq > 0 && Nc > 0 && nk > 0, NSA_ERR_ARG, "compressed scores: sizes");
  NSA_REQUIRE(cmp_block > 0 && cmp_stride > 0 && cmp_stride <= cmp_block && bn > 0, NSA_ERR_ARG, "compressed scores: block sizes");
  NSA_REQUIRE(force_first >= 0 && force_local >= 0, NSA_ERR_ARG, "compressed scores: negative forced-block counts");
  NSA_REQUIRE(cmp_scores_tc5_supports(D, dtype, cmp_block, cmp_stride, bn, nk), NSA_ERR_UNSUPPORTED,
              "compressed scores (tcgen05): needs D in {64,128}, 16-bit storage and score rows that fit shared memory (nk=%d)", nk);
  return cmp_block_scores_tc5(Q, Kc, lse, scores, head_scratch, B, H, Hkv, Tq, Nc, D, nk, cmp_block, cmp_stride, cmp_offset, bn,
                              sel_offset, causal, scale, force_first, force_local, shared_per_group, dtype, (cudaStream_t)stream);
}

int nsa_topk_from_scores(const float* scores, int32_t* idx, int BH, int nq, int nk, int top_k, int bm, int bn,
                         int offset, int causal, nsa_stream_t stream) {
  NSA_REQUIRE(scores && idx, NSA_ERR_ARG, "topk: NULL pointer");
  return topk_from_scores(scores, idx, BH, nq, nk, top_k, bm, bn, offset, causal, (cudaStream_t)stream);
}

int nsa_attention_fwd(const nsa_fwd_args* args, nsa_stream_t stream) {
  NSA_REQUIRE(args, NSA_ERR_ARG, "attention forward: NULL argument block");
  int rc = check_fwd(*args);
  if (rc != NSA_OK) return rc;
  const bool tc5 = attention_fwd_tc5_supports(*args);
  if (args->engine == NSA_ENGINE_TCGEN05) {
    NSA_REQUIRE(tc5, NSA_ERR_UNSUPPORTED, "attention forward: the tcgen05 kernel does not take this shape");
    return attention_fwd_tc5(*args, (cudaStream_t)stream);
  }
  if (args->engine == NSA_ENGINE_AUTO && tc5) {
    // One block list per query head makes the tcgen05 kernel stage the union of four lists for 256 rows of
    // which 64 use each block; measured, a selected-only launch at D=64 is then faster on the generic
    // kernel (0.99 ms against 1.90 ms at B=2, T=32768, Hq=12, Hkv=1), everything else on tcgen05.
    const bool sel_only_per_head = !args->fused && args->branches == NSA_BRANCH_SELECTED && args->Hi == args->H && args->D == 64 &&
                                   args->kv_dtype == args->q_dtype;
    // Multi-head attention (one KV head per query head) at D=64 with its per-head lists: a tcgen05 work item is then
    // four query blocks of one head, whose four lists it merges and masks, so three quarters of the selected
    // branch's MMA work is masked out; measured at B=1, T=65536, H=Hkv=16 the fused forward takes 3.05 ms on the
    // generic kernel against 3.78 ms (equal at T=4096).
    const bool mha_fused_d64 = args->fused && args->D == 64 && args->H == args->Hkv && (args->branches & NSA_BRANCH_SELECTED) &&
                               is16(args->q_dtype) && args->kv_dtype == args->q_dtype && args->accumulate == 0 &&
                               args->lse == nullptr && args->dyn_len == nullptr && args->nsplit <= 1;
    if (!sel_only_per_head && !mha_fused_d64) return attention_fwd_tc5(*args, (cudaStream_t)stream);
  }
  NSA_REQUIRE(args->dyn_len == nullptr, NSA_ERR_UNSUPPORTED, "attention forward: a device-resident length needs the tcgen05 kernel");
  NSA_REQUIRE(args->kv_dtype == args->q_dtype, NSA_ERR_UNSUPPORTED, "attention forward: bf16 K/V beside an fp8 Q need the tcgen05 kernel");
  NSA_REQUIRE(args->accumulate == 0 && !(args->fused && args->lse != nullptr), NSA_ERR_UNSUPPORTED,
              "attention forward: accumulate / lse of a fused launch need the tcgen05 kernel");
  return attention_fwd_generic(*args, (cudaStream_t)stream);
}

int nsa_device_status(nsa_stream_t stream) {
  int v = 0;
  int rc = tc5_take_status((cudaStream_t)stream, &v);
  if (rc != NSA_OK) return rc;
  int v2 = 0;
  if ((rc = cs5_take_status(&v2)) != NSA_OK) return rc;
  if (v == 0 && v2 != 0) v = 100 + v2;
  int v3 = 0;
  if ((rc = bw5_take_status(&v3)) != NSA_OK) return rc;
  if (v == 0 && v3 != 0) v = 200 + v3;
  if (v != 0) return fail(NSA_ERR_DEVICE, "a kernel gave up waiting on barrier %d (bounded wait expired)", v - 1);
  return NSA_OK;
}

int nsa_debug_set_device_status(int kernel_family, int value) {
  NSA_REQUIRE(kernel_family == 0 || kernel_family == 2, NSA_ERR_ARG, "debug status: kernel family %d (0 = forward, 2 = backward)", kernel_family);
  return kernel_family == 0 ? tc5_set_status(value) : bw5_set_status(value);
}

int launch_selected_attn_fwd(const void* Q, const void* K, const void* V, const int* Idx, void* Out, float* Lse, int BH,
                             int n_q_blocks, int Tq_p, int Tk_p, int D, int top_k, int offset, int causal,
                             float sm_scale, nsa_stream_t stream) {
  NSA_REQUIRE(Tq_p % 64 == 0 && Tk_p % 64 == 0 && n_q_blocks == Tq_p / 64, NSA_ERR_ARG,
              "launch_selected_attn_fwd: lengths must be padded to 64 (Tq_p=%d Tk_p=%d nq=%d)", Tq_p, Tk_p, n_q_blocks);
  nsa_fwd_args a = {};
  a.Q = Q; a.K = K; a.V = V; a.idx = Idx; a.out = Out; a.lse = Lse;
  a.B = 1; a.H = BH; a.Hkv = BH; a.Hi = BH;
  a.Tq = Tq_p; a.Tk = Tk_p; a.D = D; a.offset = offset;
  a.nq = n_q_blocks; a.top_k = top_k; a.bm = 64; a.bn = 64; a.sel_key_limit = Tk_p;
  a.causal = causal; a.branches = NSA_BRANCH_SELECTED; a.fused = 0;
  a.q_dtype = a.kv_dtype = NSA_BF16; a.scale = sm_scale; a.engine = NSA_ENGINE_AUTO;
  return nsa_attention_fwd(&a, stream);
}

int nsa_bwd_delta(const void* dO, const void* O, float* delta, int64_t rows, int D, int dtype, nsa_stream_t stream) {
  NSA_REQUIRE(dO && O && delta, NSA_ERR_ARG, "delta: NULL pointer");
  return bwd_delta(dO, O, delta, rows, D, dtype, (cudaStream_t)stream);
}

static int check_bwd(const nsa_bwd_args* a) {
  NSA_REQUIRE(a, NSA_ERR_ARG, "attention backward: NULL argument block");
  NSA_REQUIRE(a->Q && a->K && a->V && a->dO && a->lse && a->delta && a->dQ && a->dK_f && a->dV_f, NSA_ERR_ARG,
              "attention backward: NULL pointer");
  NSA_REQUIRE(a->B > 0 && a->H > 0 && a->Hkv > 0 && a->H % a->Hkv == 0, NSA_ERR_ARG, "attention backward: heads %d/%d", a->H, a->Hkv);
  NSA_REQUIRE(a->Tq > 0 && a->Tk > 0, NSA_ERR_ARG, "attention backward: empty problem");
  NSA_REQUIRE(a->dq_dtype == NSA_FP32 || a->dq_dtype == a->dtype, NSA_ERR_ARG, "attention backward: dQ dtype %d", a->dq_dtype);
  if (a->branch == NSA_BRANCH_SELECTED) {
    NSA_REQUIRE(a->idx, NSA_ERR_ARG, "selected backward: block index pointer is NULL");
    NSA_REQUIRE(a->Hi == a->H || a->Hi == a->Hkv, NSA_ERR_ARG, "selected backward: index heads %d", a->Hi);
    NSA_REQUIRE(a->bm > 0 && a->bn > 0 && a->top_k > 0, NSA_ERR_ARG, "selected backward: empty problem");
    NSA_REQUIRE(a->nq == (a->Tq + a->bm - 1) / a->bm, NSA_ERR_ARG, "selected backward: nq %d != ceil(Tq/bm)", a->nq);
    NSA_REQUIRE(a->sel_key_limit >= a->Tk && a->sel_key_limit < a->Tk + a->bn, NSA_ERR_ARG, "selected backward: key limit %d", a->sel_key_limit);
  } else if (a->branch == NSA_BRANCH_SLIDING) {
    NSA_REQUIRE(a->window >= 1, NSA_ERR_ARG, "sliding backward: window %d", a->window);
  } else if (a->branch == NSA_BRANCH_COMPRESSED) {
    NSA_REQUIRE(a->Nc >= 0 && a->cmp_block > 0 && a->cmp_stride > 0 && a->cmp_stride <= a->cmp_block, NSA_ERR_ARG,
                "compressed backward: Nc %d block %d stride %d", a->Nc, a->cmp_block, a->cmp_stride);
  } else {
    return fail(NSA_ERR_ARG, "attention backward: branch %d", a->branch);
  }
  return NSA_OK;
}

int nsa_attention_bwd(const nsa_bwd_args* a, nsa_stream_t stream) {
  NSA_REQUIRE(a, NSA_ERR_ARG, "attention backward: NULL argument block");
  nsa_bwd_args b = *a;
  if (b.branch == 0) b.branch = NSA_BRANCH_SELECTED;
  int rc = check_bwd(&b);
  if (rc != NSA_OK) return rc;
  if (b.branch == NSA_BRANCH_COMPRESSED && b.Nc == 0) return NSA_OK;
  NSA_REQUIRE(b.engine == NSA_ENGINE_AUTO || b.engine == NSA_ENGINE_GENERIC || b.engine == NSA_ENGINE_TCGEN05, NSA_ERR_ARG,
              "attention backward: engine %d", b.engine);
  const bool tc5 = attention_bwd_tc5_supports(b);
  if (b.engine == NSA_ENGINE_TCGEN05) {
    NSA_REQUIRE(tc5, NSA_ERR_UNSUPPORTED, "attention backward: the tcgen05 engine does not take this shape or branch");
    return attention_bwd_tc5(b, b.scratch, b.scratch_bytes, (cudaStream_t)stream);
  }
  if (b.engine == NSA_ENGINE_AUTO && tc5 && b.scratch != nullptr) return attention_bwd_tc5(b, b.scratch, b.scratch_bytes, (cudaStream_t)stream);
  return attention_bwd(b, (cudaStream_t)stream);
}

int64_t nsa_attention_bwd_scratch_bytes(const nsa_bwd_args* a) {
  NSA_REQUIRE(a, NSA_ERR_ARG, "attention backward: NULL argument block");
  nsa_bwd_args b = *a;
  if (b.branch == 0) b.branch = NSA_BRANCH_SELECTED;
  // sizes only: the pointers may still be NULL when the caller asks how much to allocate
  if (!(b.B > 0 && b.H > 0 && b.Hkv > 0 && b.H % b.Hkv == 0 && b.Tq > 0 && b.Tk > 0 && b.nq > 0 && b.top_k > 0)) return 0;
  if (!attention_bwd_tc5_supports(b)) return 0;
  return attention_bwd_tc5_scratch_bytes(b);
}

int nsa_selected_bwd(const nsa_bwd_args* a, nsa_stream_t stream) {
  NSA_REQUIRE(a, NSA_ERR_ARG, "selected backward: NULL argument block");
  nsa_bwd_args b = *a;
  b.branch = NSA_BRANCH_SELECTED;
  return nsa_attention_bwd(&b, stream);
}

int nsa_pool_mean_bwd(const float* dxc, float* dx, int B, int H, int T, int D, int block, int stride, int n_out,
                      nsa_stream_t stream) {
  NSA_REQUIRE(dxc && dx, NSA_ERR_ARG, "pool backward: NULL pointer");
  return pool_mean_bwd(dxc, dx, B, H, T, D, block, stride, n_out, (cudaStream_t)stream);
}

int launch_selected_attn_bwd(const void* Q, const void* K, const void* V, const void* dO, const float* LSE,
                             const float* Dvec, const int* Idx, void* dQ, float* dK_f, float* dV_f, int BH,
                             int n_q_blocks, int Tq_p, int Tk_p, int D, int top_k, int offset, int causal,
                             float sm_scale, nsa_stream_t stream) {
  NSA_REQUIRE(Tq_p % 64 == 0 && Tk_p % 64 == 0 && n_q_blocks == Tq_p / 64, NSA_ERR_ARG,
              "launch_selected_attn_bwd: lengths must be padded to 64 (Tq_p=%d Tk_p=%d nq=%d)", Tq_p, Tk_p, n_q_blocks);
  nsa_bwd_args a = {};
  a.Q = Q; a.K = K; a.V = V; a.dO = dO; a.lse = LSE; a.delta = Dvec; a.idx = Idx;
  a.dQ = dQ; a.dK_f = dK_f; a.dV_f = dV_f;
  a.B = 1; a.H = BH; a.Hkv = BH; a.Hi = BH; a.Tq = Tq_p; a.Tk = Tk_p; a.D = D;
  a.nq = n_q_blocks; a.top_k = top_k; a.bm = 64; a.bn = 64; a.sel_key_limit = Tk_p;
  a.offset = offset; a.causal = causal; a.dtype = NSA_BF16; a.dq_dtype = NSA_BF16; a.scale = sm_scale;
  a.branch = NSA_BRANCH_SELECTED;
  const int64_t need = nsa_attention_bwd_scratch_bytes(&a);
  if (need <= 0) return nsa_selected_bwd(&a, stream);
  void* scratch = nullptr;
  NSA_CUDA_OK(cudaMallocAsync(&scratch, (size_t)need, (cudaStream_t)stream));
  a.scratch = scratch;
  a.scratch_bytes = need;
  const int rc = nsa_selected_bwd(&a, stream);
  NSA_CUDA_OK(cudaFreeAsync(scratch, (cudaStream_t)stream));
  return rc;
}

int nsa_combine(const void* out_c, const void* out_s, const void* out_w, const void* gates, void* out, int64_t rows,
                int D, int activation, int dtype, int gate_dtype, nsa_stream_t stream) {
  NSA_REQUIRE(out_c && out_s && out_w && gates && out, NSA_ERR_ARG, "combine: NULL pointer");
  return combine(out_c, out_s, out_w, gates, out, rows, D, activation, dtype, gate_dtype, (cudaStream_t)stream);
}

int nsa_fp8_absmax(const void* x, int64_t n, int dtype, float* absmax, nsa_stream_t stream) {
  NSA_REQUIRE(x && absmax, NSA_ERR_ARG, "absmax: NULL pointer");
  return fp8_absmax(x, n, dtype, absmax, (cudaStream_t)stream);
}

int nsa_fp8_quantize(const void* x, void* out8, int64_t n, int dtype, int fmt, float scale, nsa_stream_t stream) {
  NSA_REQUIRE(x && out8, NSA_ERR_ARG, "quantize: NULL pointer");
  return fp8_quantize(x, out8, n, dtype, fmt, scale, (cudaStream_t)stream);
}

int nsa_fp8_dequantize(const void* x8, void* out, int64_t n, int fmt, float scale, nsa_stream_t stream) {
  NSA_REQUIRE(x8 && out, NSA_ERR_ARG, "dequantize: NULL pointer");
  NSA_REQUIRE(n >= 0, NSA_ERR_ARG, "dequantize: n=%lld", (long long)n);
  return fp8_dequantize(x8, out, n, fmt, scale, (cudaStream_t)stream);
}

int nsa_cast_from_f32(const float* src, void* dst, int64_t n, int dtype, nsa_stream_t stream) {
  NSA_REQUIRE(src && dst, NSA_ERR_ARG, "cast: NULL pointer");
  return cast_from_f32(src, dst, n, dtype, (cudaStream_t)stream);
}

int nsa_rope_to_heads(const void* x, void* y, const void* cos, const void* sin, int B, int T, int H, int D, int x_dtype,
                      int cs_dtype, int y_dtype, nsa_stream_t stream) {
  NSA_REQUIRE(x && y, NSA_ERR_ARG, "rope_to_heads: NULL pointer");
  NSA_REQUIRE((cos == nullptr) == (sin == nullptr), NSA_ERR_ARG, "rope_to_heads: cos and sin must both be given or both be NULL");
  NSA_REQUIRE(B >= 0 && T >= 0 && H > 0 && D > 0, NSA_ERR_ARG, "rope_to_heads: bad sizes B=%d T=%d H=%d D=%d", B, T, H, D);
  NSA_REQUIRE(D % 16 == 0, NSA_ERR_UNSUPPORTED, "rope_to_heads: D=%d must be a multiple of 16", D);
  NSA_REQUIRE(x_dtype == NSA_FP32 || x_dtype == NSA_BF16 || x_dtype == NSA_FP16, NSA_ERR_UNSUPPORTED, "rope_to_heads: x dtype %d", x_dtype);
  NSA_REQUIRE(y_dtype == NSA_BF16 || y_dtype == NSA_FP16, NSA_ERR_UNSUPPORTED, "rope_to_heads: y dtype %d must be 16-bit", y_dtype);
  NSA_REQUIRE(cos == nullptr || cs_dtype == NSA_FP32 || cs_dtype == NSA_BF16 || cs_dtype == NSA_FP16, NSA_ERR_UNSUPPORTED,
              "rope_to_heads: cos/sin dtype %d", cs_dtype);
  return rope_to_heads(x, y, cos, sin, B, T, H, D, x_dtype, cs_dtype, y_dtype, (cudaStream_t)stream);
}

int nsa_cache_append(const void* k_new, const void* v_new, void* K, void* V, void* Kc, void* Vc, void* Kb, int B, int Hkv, int D,
                     int t_new, int filled, int max_len, int nc_alloc, int nb_alloc, int cmp_block, int cmp_stride, int sel_block,
                     int dtype, nsa_stream_t stream) {
  NSA_REQUIRE(k_new && v_new && K && V && Kc && Vc && Kb, NSA_ERR_ARG, "cache append: NULL pointer");
  return cache_append(k_new, v_new, K, V, Kc, Vc, Kb, B, Hkv, D, t_new, filled, nullptr, max_len, nc_alloc, nb_alloc, cmp_block,
                      cmp_stride, sel_block, dtype, (cudaStream_t)stream);
}

int nsa_cache_append_dev(const void* k_new, const void* v_new, void* K, void* V, void* Kc, void* Vc, void* Kb, int B, int Hkv, int D,
                         int t_new, int32_t* filled, int max_len, int nc_alloc, int nb_alloc, int cmp_block, int cmp_stride,
                         int sel_block, int dtype, nsa_stream_t stream) {
  NSA_REQUIRE(k_new && v_new && K && V && Kc && Vc && Kb && filled, NSA_ERR_ARG, "cache append: NULL pointer");
  return cache_append(k_new, v_new, K, V, Kc, Vc, Kb, B, Hkv, D, t_new, 0, filled, max_len, nc_alloc, nb_alloc, cmp_block,
                      cmp_stride, sel_block, dtype, (cudaStream_t)stream);
}

int nsa_memcpy_2d(void* dst, size_t dst_pitch, const void* src, size_t src_pitch, size_t row_bytes, size_t rows,
                  int to_device, nsa_stream_t stream) {
  NSA_REQUIRE(dst && src, NSA_ERR_ARG, "memcpy_2d: NULL pointer");
  NSA_REQUIRE(to_device == 0 || to_device == 1, NSA_ERR_ARG, "memcpy_2d: to_device must be 0 or 1");
  NSA_REQUIRE(dst_pitch >= row_bytes && src_pitch >= row_bytes, NSA_ERR_ARG, "memcpy_2d: pitch smaller than a row");
  if (row_bytes == 0 || rows == 0) return NSA_OK;
  NSA_CUDA_OK(cudaMemcpy2DAsync(dst, dst_pitch, src, src_pitch, row_bytes, rows,
                                to_device ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToHost, (cudaStream_t)stream));
  return NSA_OK;
}

}  // extern "C"
