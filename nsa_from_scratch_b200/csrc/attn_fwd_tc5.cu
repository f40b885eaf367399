// NSA attention forward on the 5th-generation tensor cores (tcgen05 + TMEM + TMA), sm_100a.
//
// Work item = (batch, KV head, 4 query heads of its group, one 64-position query block):
// 256 rows = two 128-row MMA tiles (tile X holds heads 2X and 2X+1 of the quad, 64 positions each).
// All rows of a work item see the same KV tiles in every branch (the selected blocks are
// shared by the heads of a GQA group), so a K/V tile staged once by TMA feeds both tiles.
//
// Warp roles (12 warps launched at 168 registers, one block per SM; with setmaxnreg warps 0-3 shrink to
// 72 and the 8 softmax warps grow to 216.  What the .inc calls take must have been released by .dec
// calls of the SAME block -- 8*(216-168) <= 4*(168-72) -- otherwise setmaxnreg.inc blocks forever):
//   warp 0      TMA producer: Q once, then K and V tiles (1 or 2 chunks of 64 keys) into two
//               2-deep rings of 128-byte-swizzled shared memory; pooled K/V for the compressed
//               branch, raw K/V for the selected and sliding branches
//   warp 1      MMA issuer (one thread): S_X = Q_X K^T into TMEM, then O_X (+)= P_X V with P read
//               from TMEM (it aliases S_X) and V as an MN-major shared-memory operand
//   warps 4-7   softmax of tile 0, warps 8-11 softmax of tile 1 (one thread per row; a warp reaches
//               the TMEM lanes 32*(warp%4)..+31): read the whole S row from TMEM in one round trip,
//               mask, running max with lazy rescale of O (only when the max grows by > 2^8), exp2,
//               row sum, P as 16-bit back into TMEM; at the end of a branch they read O, apply
//               gate/l and add it into the output row (the row itself holds the running gated sum)
// TMEM columns: S0 [0,128) S1 [128,256) O0 [256,256+D) O1 [384,384+D).
// Tile X's chain QK -> softmax -> PV is serial; the tensor pipe stays busy because the other
// tile's MMAs run in the gaps.  Every mbarrier wait is bounded; a wait that gives up raises a
// block-wide abort flag, sets the device status word and the block still frees its TMEM.
#include "common.cuh"
#include "tc5_ptx.cuh"

#include <cudaTypedefs.h>
#include <stdlib.h>

namespace nsa {

using namespace tc5;

constexpr int T5_MAX_SEL = 64;            // listed blocks per query block
constexpr int T5_MAX_ENT = 4 * T5_MAX_SEL;  // entries of the four row groups of a work item
constexpr int T5_THREADS = 384;   // 12 warps; register budget rebalanced per role with setmaxnreg

__device__ int g_tc5_status;   // 0 ok; otherwise (1 + id of the barrier a wait gave up on)

struct Tc5Params {
  CUtensorMap tmQ, tmK, tmV, tmKc, tmVc;
  CUtensorMap tmOf;  // one-item kernel: the output in boxes of 32 positions x 64 elements of one head, 128-byte swizzle (an item's last write)
  CUtensorMap tmO;   // persistent kernel: the output, 4-D in the order of its strides, boxes of 32 positions x 32 elements of one head, 64-byte swizzle
  nsa_fwd_args a;
  float scale_log2[3];   // per branch: softmax scale * log2(e) (* the fp8 dequantisation scales of the operands)
  float out_scale[3];    // per branch: factor on P.V (the fp8 scale of V; 1 otherwise)
  int nk_blocks;
  int GH;          // query heads per work item (4, 2 or 1); a work item has 4/GH consecutive query blocks
  int HG;          // head groups per KV head = (H/Hkv) / GH
  int NQG;         // query-block groups = ceil(nq / (4/GH))
  int nsplit;      // split launches: thread blocks per work item, each with a share of every branch's key tiles
  float* part;     // split launches: partial results [B*H*Tq][nsplit][3][D+4] = unnormalised O, m (log2 units), l
  int kv8;         // fp8 launches: K/V are fp8 too (converted tile by tile); 0 = K/V arrive as bf16, only Q is fp8
  int tma_out;     // persistent kernel: an item whose result is ONE branch writes it through shared memory and the TMA (rows_through_tma)
  int fin_tma;     // one-item kernel, D = 128: the item's last branch end writes the output rows through shared memory and two TMA boxes per warp
  int psum;        // one-item kernel, unsplit 16-bit launches: 32 KB of shared memory hold the first 64 columns of the rows' running gated sum
  int poly;        // tiles without masked entries take 3 of every 8 exponentials on the FMA pipe (exp2_poly_pair)
};

struct Tile {
  int nch;
  int j0[2];
  int jlim[2];
  int mask[2];   // which of the 4 row groups attend the chunk (selected branch; 0xF otherwise)
};

// Row maximum (raw scores) of the 64 * nch columns a softmax thread holds: four chains of 3-input max.
__device__ __forceinline__ float row_max_raw(const uint32_t (&sv)[4][32], int nch) {
  float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
  for (int g = 0; g < 2; ++g)
#pragma unroll
    for (int i = 0; i < 32; i += 2) m4[(i >> 1) & 3] = max3(m4[(i >> 1) & 3], __uint_as_float(sv[g][i]), __uint_as_float(sv[g][i + 1]));
  if (nch == 2) {
#pragma unroll
    for (int g = 2; g < 4; ++g)
#pragma unroll
      for (int i = 0; i < 32; i += 2) m4[(i >> 1) & 3] = max3(m4[(i >> 1) & 3], __uint_as_float(sv[g][i]), __uint_as_float(sv[g][i + 1]));
  }
  return fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
}

// P = exp2(S * sl2 - m_ref) for 32 columns of a row without masked entries, as 16 packed 16-bit pairs; the row sums
// go to the packed accumulators.  Of every 8 pairs, 3 are evaluated by the polynomial on the FMA pipe and 5 by ex2 on
// the special-function unit: alone, a warp's sweep of 128 columns is bound by that unit (1024 of 1190 clocks); mixed
// this way it measured 947 clocks, and 2040 instead of 2410 with two warps sharing a scheduler.
template <typename T>
__device__ __forceinline__ void exp_group_mixed(const uint32_t (&s)[32], f32x2 SL, f32x2 NM, f32x2& sa, f32x2& sb, uint32_t (&pk)[16]) {
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const f32x2 x = fma2(mk2(__uint_as_float(s[2 * i]), __uint_as_float(s[2 * i + 1])), SL, NM);
    float p0, p1;
    if ((i & 7) < 3) {
      exp2_poly_pair(x, p0, p1);
    } else {
      float x0, x1;
      un2(x, x0, x1);
      p0 = ex2(x0);
      p1 = ex2(x1);
    }
    const f32x2 pp = mk2(p0, p1);
    if (i & 1) sb = add2(sb, pp); else sa = add2(sa, pp);
    pk[i] = Elem<T>::pack(p0, p1);
  }
}

// End of a branch that alone makes up an item's result (single-branch launches), for one softmax warp: its 32 rows of
// O (one thread per row in TMEM, D fp32 columns at tO) times the rows' coefficients, rounded to 16 bits, leave through a
// 2 KB staging box (32 rows x 32 elements, 64-byte swizzle: 16-byte piece k of row r sits at piece k ^ ((r >> 1) & 3),
// which also keeps the lanes' writes off each other's banks) and TMA stores.  A thread writing its own row with
// 16-byte stores touches 32 lines per instruction; this way the load/store unit is not involved and the values are
// the same.  The TMA takes about 100 clocks per box instruction and SM, so this pays only where nothing has to be
// read back: with several branches per item every variant tried (16-bit adds in L2, fp32 sums in an L2-resident
// slot, transposing through shared memory) lost to the per-row code or to the 2e-2 bound.
// Rows past Tq are clipped by the tensor map.  `issue(smem address, first column)` starts the copy of one box.
template <typename T, int D, typename Issue>
__device__ __forceinline__ void rows_through_tma(unsigned char* stage, uint32_t tO, float coef, int lane, Issue issue) {
  const int sw = (lane >> 1) & 3;
#pragma unroll
  for (int c = 0; c < D / 32; ++c) {
    uint32_t v[32];
    tmem_ld32(tO + c * 32, v);
    tc_wait_ld();
    uint32_t w[16];
#pragma unroll
    for (int e = 0; e < 16; ++e) w[e] = Elem<T>::pack(__uint_as_float(v[2 * e]) * coef, __uint_as_float(v[2 * e + 1]) * coef);
    if (lane == 0) bulk_wait_read<0>();             // the box issued before has been read out of the staging area
    __syncwarp();
#pragma unroll
    for (int k = 0; k < 4; ++k)
      *reinterpret_cast<uint4*>(stage + lane * 64 + ((k ^ sw) << 4)) = make_uint4(w[4 * k], w[4 * k + 1], w[4 * k + 2], w[4 * k + 3]);
    fence_proxy_async();
    __syncwarp();
    if (lane == 0) {
      issue(smem_u32(stage), c * 32);
      bulk_commit();
    }
  }
}

// barrier ids
enum { B_QFULL = 0, B_KFULL = 1, B_KEMPTY = 3, B_VFULL = 5, B_VEMPTY = 7, B_SFULL = 9, B_PFULL = 11, B_PVDONE = 13,
       B_STGFULL = 15, B_STGEMPTY = 17, B_SREAD = 19, B_PHALF = 21, B_COUNT = 23 };
// STG*: fp8 staging buffers (0 = K side, 1 = V side); SREAD: D=64 only, "S row is in registers";
// PHALF: D=128, one-item kernel: "P of the tile's first 64 keys is in TMEM" -- that half of P V is issued while the second
// half of the exponentials is still being computed, which takes it off the tile's QK -> softmax -> PV chain

// SPLIT: decoding-sized launches (few work items, long key ranges).  nsplit thread blocks share a work item; block s
// takes tiles [nt*s/nsplit, nt*(s+1)/nsplit) of each branch and leaves (unnormalised O, m, l) per branch and row
// in p.part; nsa_split_combine_kernel merges them and applies the gates.
template <int D, int FMT, bool IN8, bool SPLIT>
__global__ void __launch_bounds__(384, 1) nsa_fwd_tc5_kernel(const __grid_constant__ Tc5Params p) {
  using T = typename std::conditional<FMT == 1, __nv_bfloat16, __half>::type;
  constexpr int DH = D / 64;                    // 64-element (128-byte) halves of a row
  constexpr int QTILE = DH * 128 * 128;         // bytes of one 128-row Q tile
  constexpr int KVTILE = DH * 128 * 128;        // bytes of one 128-key K or V tile
  constexpr int DHSTRIDE = 128 * 128;           // bytes between the halves
  // D = 64 leaves 64 TMEM columns per tile unused: P gets columns of its own there instead of aliasing S,
  // so the next tile's QK^T can be issued as soon as the softmax threads hold the S row in registers
  // (not only after PV has consumed P) -- the QK -> softmax -> PV chain of a tile is broken.
  constexpr bool EARLY = (D == 64);
  const nsa_fwd_args& a = p.a;

  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sQ = smem_u32(smem);
  const uint32_t sK = sQ + 2 * QTILE;
  const uint32_t sV = sK + 2 * KVTILE;
  // fp8 storage only: two staging buffers of 128 rows x D bytes (plain row-major), filled by TMA and turned
  // into the swizzled 16-bit tiles above by warps 2 (K side) and 3 (V side); Q goes through them first
  constexpr int STG = 128 * D;
  unsigned char* stg = smem + 2 * QTILE + 4 * KVTILE;
  __shared__ __align__(8) uint64_t bars[B_COUNT];
  __shared__ int sel_list[T5_MAX_ENT];            // selected branch: key blocks to visit ...
  __shared__ unsigned char sel_mask[T5_MAX_ENT];  // ... and the row groups that listed each of them
  __shared__ int sel_n;
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_flag;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  // ---- work item -------------------------------------------------------------------
  // 4 row groups of 64 query positions: group g = (head h_base + g % GH, query block qb_base + g / GH);
  // MMA tile X holds groups 2X and 2X+1.
  const int per_q = a.B * a.Hkv * p.HG;
  const unsigned item = SPLIT ? blockIdx.x / (unsigned)p.nsplit : blockIdx.x;
  const int split = SPLIT ? (int)(blockIdx.x % (unsigned)p.nsplit) : 0;
  const int qbg = p.NQG - 1 - (int)(item / per_q);   // long rows first
  const int rem = (int)(item % per_q);
  const int b = rem / (a.Hkv * p.HG);
  const int hk = (rem / p.HG) % a.Hkv;
  const int hg = rem % p.HG;
  const int G = a.H / a.Hkv;
  const int GH = p.GH, NQB = 4 / p.GH;
  const int h_base = hk * G + hg * GH;
  const int qb_base = qbg * NQB;
  auto grp_head = [&](int g) { return h_base + g % GH; };
  auto grp_qb = [&](int g) { return qb_base + g / GH; };
  const int q_first = qb_base * 64;
  const int i_last = min((min(qb_base + NQB, a.nq)) * 64, a.Tq) - 1;
  const int kv_slab = b * a.Hkv + hk;

  auto bar = [&](int id) { return smem_u32(&bars[id]); };

  // Length-dependent launch parameters.  Split (decoding) launches may take the number of filled key positions
  // from device memory (a.dyn_len), so that a captured CUDA graph of a decoding step stays valid as the cache
  // grows; everything else reads the launch parameters as they are.
  int dyn_off = 0, dyn_cmp_off = 0, dyn_sel_lim = 0;
  if constexpr (SPLIT) {
    if (a.dyn_len != nullptr) {
      const int len = *a.dyn_len;
      dyn_off = len - a.Tq;
      dyn_cmp_off = (a.cmp_stride == a.cmp_block ? (len + a.cmp_block - 1) / a.cmp_block * a.cmp_block : len) - a.Tq;
      dyn_sel_lim = (len + 63) / 64 * 64;
    }
  }
  auto OFFSET = [&]() { if constexpr (SPLIT) return a.dyn_len != nullptr ? dyn_off : a.offset; else return a.offset; };
  auto CMP_OFFSET = [&]() { if constexpr (SPLIT) return a.dyn_len != nullptr ? dyn_cmp_off : a.cmp_offset; else return a.cmp_offset; };
  auto SEL_LIMIT = [&]() { if constexpr (SPLIT) return a.dyn_len != nullptr ? dyn_sel_lim : a.sel_key_limit; else return a.sel_key_limit; };

  // ---- per-branch key bounds of a query row -------------------------------------------
  auto bounds = [&](int br, int i, bool ok, int& lo, int& hi) {
    lo = 0; hi = -1;
    if (!ok) return;
    if (br == 0) {
      if (a.causal) {
        int num = i + CMP_OFFSET() - (a.cmp_block - 1);
        hi = num < 0 ? -1 : num / a.cmp_stride;
      } else hi = a.Nc - 1;
      hi = min(hi, a.Nc - 1);
    } else if (br == 1) {
      hi = a.causal ? min(i + OFFSET(), SEL_LIMIT() - 1) : SEL_LIMIT() - 1;
    } else {
      int pos = i + OFFSET();
      if (a.causal) { lo = pos - a.window + 1; hi = pos; }
      else { lo = pos - a.window; hi = pos + a.window; }
      lo = max(lo, 0); hi = min(hi, a.Tk - 1);
    }
  };

  // ---- setup: barriers, TMEM, list of selected blocks ---------------------------------------
  if (tid == 0) {
    abort_flag = 0;
    for (int i = 0; i < B_COUNT; ++i)
      mbar_init(bar(i), (i == B_PFULL || i == B_PFULL + 1 || i == B_SREAD || i == B_SREAD + 1 || i == B_PHALF || i == B_PHALF + 1) ? 128 : ((IN8 && i == B_QFULL) ? 2 : 1));
    fence_barrier_init();
  }
  if (warp == 1) { tmem_alloc(smem_u32(&tmem_base_s), 512); tmem_relinquish(); }
  // scratch of the list builder: the first bytes of the (not yet used) Q tile area
  int* ent_blk = reinterpret_cast<int*>(smem);
  unsigned char* ent_p = smem + T5_MAX_ENT * sizeof(int);
  if (warp == 2) {
    // Selected branch: the key blocks the work item visits, each with the set of row groups that list it.
    // Lists shared by the 4 groups (one list per KV head, GH == 4) are taken as they are.  Otherwise the
    // 4 lists are merged: a block listed by several groups is staged once and masked per group; a block
    // listed p times by one group is visited p times (the reference counts duplicates twice).
    int n = 0;
    if (a.branches & NSA_BRANCH_SELECTED) {
      const bool shared = a.Hi != a.H && GH == 4;
      const int ngrp = shared ? 1 : 4;
      const int n_ent = ngrp * a.top_k;
      for (int i = lane; i < n_ent; i += 32) {
        const int g = i / a.top_k, sl = i % a.top_k;
        const int qb = grp_qb(g);
        int blk = -1;
        if (qb < a.nq) {
          const int hi_ = (a.Hi == a.H) ? grp_head(g) : hk;
          blk = a.idx[(((size_t)b * a.Hi + hi_) * a.nq + qb) * a.top_k + sl];
          const int last_pos = min(qb * 64 + 64, a.Tq) - 1 + OFFSET();
          if (blk < 0 || blk >= SEL_LIMIT() / 64 || (a.causal && (long long)blk * 64 > last_pos)) blk = -1;
        }
        ent_blk[i] = blk;
      }
      __syncwarp();
      if (!shared) {
        for (int i = lane; i < n_ent; i += 32) {          // p = how many earlier entries of the same group list the same block
          int pc = 0;
          const int blk = ent_blk[i], g0 = (i / a.top_k) * a.top_k;
          for (int j = g0; j < i; ++j) pc += (ent_blk[j] == blk);
          ent_p[i] = (unsigned char)pc;
        }
        __syncwarp();
      }
      for (int i0 = 0; i0 < n_ent; i0 += 32) {
        const int i = i0 + lane;
        bool lead = false;
        unsigned msk = 0xFu;
        if (i < n_ent && ent_blk[i] >= 0) {
          lead = true;
          if (!shared) {
            const int blk = ent_blk[i], pi = ent_p[i], gi = i / a.top_k;
            msk = 0;
            for (int j = 0; j < n_ent; ++j) {
              if (ent_blk[j] == blk && ent_p[j] == pi) {
                const int gj = j / a.top_k;
                msk |= 1u << gj;
                if (gj < gi) lead = false;
              }
            }
          }
        }
        const unsigned bal = __ballot_sync(0xffffffffu, lead);
        if (lead) {
          const int pos = n + __popc(bal & ((1u << lane) - 1));
          sel_list[pos] = ent_blk[i];
          sel_mask[pos] = (unsigned char)msk;
        }
        n += __popc(bal);
      }
    }
    if (lane == 0) sel_n = n;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_s;

  // chunk counts of the three branches (uniform over the block)
  int nchunks[3] = {0, 0, 0};
  int sld_c0 = 0;
  {
    int lo_f, hi_f, lo_l, hi_l;
    if (a.branches & NSA_BRANCH_COMPRESSED) {
      bounds(0, i_last, true, lo_l, hi_l);
      nchunks[0] = hi_l < 0 ? 0 : hi_l / 64 + 1;
    }
    if (a.branches & NSA_BRANCH_SELECTED) nchunks[1] = sel_n;
    if (a.branches & NSA_BRANCH_SLIDING) {
      bounds(2, q_first, true, lo_f, hi_f);
      bounds(2, i_last, true, lo_l, hi_l);
      if (hi_l >= lo_f) { sld_c0 = lo_f / 64; nchunks[2] = hi_l / 64 - sld_c0 + 1; }
    }
  }
  // tiles [tbeg(br), tend(br)) of each branch are this block's: all of them unless the launch is split
  auto tbeg = [&](int br) {
    if constexpr (SPLIT) return ((nchunks[br] + 1) >> 1) * split / p.nsplit;
    else return 0;
  };
  auto tend = [&](int br) {
    if constexpr (SPLIT) return ((nchunks[br] + 1) >> 1) * (split + 1) / p.nsplit;
    else return (nchunks[br] + 1) >> 1;
  };
  auto get_tile = [&](int br, int t) {
    Tile tl;
    tl.nch = min(2, nchunks[br] - 2 * t);
    for (int c = 0; c < 2; ++c) {
      int ci = min(2 * t + c, nchunks[br] - 1);
      tl.mask[c] = 0xF;
      if (br == 0) { tl.j0[c] = ci * 64; tl.jlim[c] = a.Nc; }
      else if (br == 1) { int blk = sel_list[ci]; tl.j0[c] = blk * 64; tl.jlim[c] = min(blk * 64 + 64, SEL_LIMIT()); tl.mask[c] = sel_mask[ci]; }
      else { tl.j0[c] = (sld_c0 + ci) * 64; tl.jlim[c] = a.Tk; }
    }
    return tl;
  };
  int fail_id = 0;   // barrier id (+1) this thread gave up on
  int last_k_it = -1, last_v_it = -1;   // producer: last tile whose K / V copies were issued
  int last_u8 = -1;                     // producer (fp8): last use of the staging buffers that was issued

  if (warp == 0) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 72;\n");
    // =============================== TMA producer ===============================
    // The whole warp walks the tile sequence (converged); one elected lane issues the copies.
    {
      const bool leader = elect_one();
      if (leader) {
        tma_prefetch_desc(&p.tmQ); tma_prefetch_desc(&p.tmK); tma_prefetch_desc(&p.tmV);
        if (a.branches & NSA_BRANCH_COMPRESSED) { tma_prefetch_desc(&p.tmKc); tma_prefetch_desc(&p.tmVc); }
        if constexpr (IN8) {
          last_u8 = 0;
          // Q tile X (2 heads x 64 positions, D bytes per row) into staging buffer X
          for (int X = 0; X < 2; ++X) {
            mbar_expect_tx(bar(B_STGFULL + X), STG);
            for (int hh = 0; hh < 2; ++hh)
              tma_load_3d(smem_u32(stg) + X * STG + hh * 64 * D, &p.tmQ, bar(B_STGFULL + X), 0, grp_qb(2 * X + hh) * 64,
                          b * a.H + grp_head(2 * X + hh));
          }
        } else {
          mbar_expect_tx(bar(B_QFULL), 2 * QTILE);
          for (int X = 0; X < 2; ++X)
            for (int hh = 0; hh < 2; ++hh)
              for (int dh = 0; dh < DH; ++dh)
                tma_load_3d(sQ + X * QTILE + dh * DHSTRIDE + hh * 8192, &p.tmQ, bar(B_QFULL), dh * 64, grp_qb(2 * X + hh) * 64,
                            b * a.H + grp_head(2 * X + hh));
        }
      }
      __syncwarp();
      int it = 0;          // tile counter over all branches
      int u8 = 1;          // fp8: use counter of the staging buffers (use 0 was Q)
      bool ok = true;
      for (int br = 0; br < 3 && ok; ++br) {
        const CUtensorMap* mk = br == 0 ? &p.tmKc : &p.tmK;
        const CUtensorMap* mv = br == 0 ? &p.tmVc : &p.tmV;
        const bool raw8 = IN8 && br != 0 && p.kv8;   // pooled K/V of the compressed branch are 16-bit already
        for (int t = tbeg(br); t < tend(br) && ok; ++t, ++it) {
          const Tile tl = get_tile(br, t);
          const int s = it & 1, ph = (it >> 1) & 1;
          if (raw8) {
            // fp8 K/V: TMA fills the staging buffers; the converter warps own the ring slots
            for (int side = 0; side < 2 && ok; ++side) {
              ok = __all_sync(0xffffffffu, mbar_wait(bar(B_STGEMPTY + side), (u8 - 1) & 1, &abort_flag));
              if (!ok) { fail_id = B_STGEMPTY + side + 1; break; }
              if (leader) {
                mbar_expect_tx(bar(B_STGFULL + side), (uint32_t)tl.nch * 64 * D);
                for (int c = 0; c < tl.nch; ++c)
                  tma_load_3d(smem_u32(stg) + side * STG + c * 64 * D, side == 0 ? mk : mv, bar(B_STGFULL + side), 0, tl.j0[c], kv_slab);
              }
            }
            last_u8 = u8;
            ++u8;
            __syncwarp();
            continue;
          }
          const uint32_t bytes = (uint32_t)tl.nch * 64 * D * 2;
          ok = __all_sync(0xffffffffu, mbar_wait(bar(B_KEMPTY + s), ph ^ 1, &abort_flag));
          if (!ok) { fail_id = B_KEMPTY + s + 1; break; }
          if (leader) {
            mbar_expect_tx(bar(B_KFULL + s), bytes);
            for (int c = 0; c < tl.nch; ++c)
              for (int dh = 0; dh < DH; ++dh)
                tma_load_3d(sK + s * KVTILE + dh * DHSTRIDE + c * 8192, mk, bar(B_KFULL + s), dh * 64, tl.j0[c], kv_slab);
          }
          last_k_it = it;
          ok = __all_sync(0xffffffffu, mbar_wait(bar(B_VEMPTY + s), ph ^ 1, &abort_flag));
          if (!ok) { fail_id = B_VEMPTY + s + 1; break; }
          if (leader) {
            mbar_expect_tx(bar(B_VFULL + s), bytes);
            for (int c = 0; c < tl.nch; ++c)
              for (int dh = 0; dh < DH; ++dh)
                tma_load_3d(sV + s * KVTILE + dh * DHSTRIDE + c * 8192, mv, bar(B_VFULL + s), dh * 64, tl.j0[c], kv_slab);
          }
          last_v_it = it;
          __syncwarp();
        }
      }
    }
  } else if (warp == 1) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 72;\n");
    // =============================== MMA issuer ===============================
    // The whole warp walks the tile sequence converged; one elected lane issues the MMAs and commits.
    // Everything an MMA needs beyond an add is computed before the loop.
    {
      const bool leader = elect_one();
      constexpr uint32_t IDESC_PV = idesc_f16(FMT, 128, D, 0, 1);
      constexpr uint32_t IDESC_QK1 = idesc_f16(FMT, 128, 64, 0, 0);
      constexpr uint32_t IDESC_QK2 = idesc_f16(FMT, 128, 128, 0, 0);
      bool ok = __all_sync(0xffffffffu, mbar_wait(bar(B_QFULL), 0, &abort_flag));
      if (!ok) fail_id = B_QFULL + 1;
      // tile counts per branch and in total; (cur_br, cur_t) walk the flattened sequence
      int nt_of[3], total_tiles = 0;
#pragma unroll
      for (int br = 0; br < 3; ++br) { nt_of[br] = tend(br) - tbeg(br); total_tiles += nt_of[br]; }
      // descriptor bases: the low word carries the address field, so "+ (bytes >> 4)" moves the start
      const uint64_t dQ[2] = {smem_desc_sw128(sQ, 16, 1024), smem_desc_sw128(sQ + QTILE, 16, 1024)};
      const uint64_t dK[2] = {smem_desc_sw128(sK, 16, 1024), smem_desc_sw128(sK + KVTILE, 16, 1024)};
      const uint64_t dV[2] = {smem_desc_sw128(sV, DHSTRIDE, 1024), smem_desc_sw128(sV + KVTILE, DHSTRIDE, 1024)};
      const uint32_t tSx[2] = {tmem, tmem + 128}, tOx[2] = {tmem + 256, tmem + 384};
      const uint32_t tPx[2] = {EARLY ? tmem + 320 : tmem, EARLY ? tmem + 448 : tmem + 128};

      // position of the tile whose QK is issued next / whose PV is issued next (tile tbeg(br) + t of the branch)
      int q_br = 0, q_t = 0, p_br = 0, p_t = 0;
      auto skip_empty = [&](int& br, int& t) { while (br < 3 && t >= nt_of[br]) { ++br; t = 0; } };
      skip_empty(q_br, q_t);
      skip_empty(p_br, p_t);

      auto issue_qk = [&](int X, int it) {          // uses (q_br, q_t); the caller advances them after X == 1
        const int nch = min(2, nchunks[q_br] - 2 * (tbeg(q_br) + q_t));
        const int s = it & 1;
        if (X == 0) {
          if (!__all_sync(0xffffffffu, mbar_wait(bar(B_KFULL + s), (it >> 1) & 1, &abort_flag))) { fail_id = B_KFULL + s + 1; return false; }
          tc_fence_after();
        }
        const uint32_t idesc = nch == 2 ? IDESC_QK2 : IDESC_QK1;
        if (leader) {
#pragma unroll
          for (int ks = 0; ks < D / 16; ++ks) {
            const uint32_t off = (uint32_t)(((ks >> 2) * DHSTRIDE + (ks & 3) * 32) >> 4);
            if (ks == 0) mma_ss(tSx[X], dQ[X] + off, dK[s] + off, idesc, 0u);
            else mma_ss(tSx[X], dQ[X] + off, dK[s] + off, idesc, 1u);
          }
          tc_commit(bar(B_SFULL + X));
          if (X == 1) tc_commit(bar(B_KEMPTY + s));
        }
        __syncwarp();
        return true;
      };
      if (ok && total_tiles > 0) {
        ok = issue_qk(0, 0) && issue_qk(1, 0);
        ++q_t; skip_empty(q_br, q_t);
      }
      for (int it = 0; it < total_tiles && ok; ++it) {
        const int nch = min(2, nchunks[p_br] - 2 * (tbeg(p_br) + p_t));
        const bool fresh = p_t == 0;                       // first tile of a branch starts a new O
        const int s = it & 1;
        ok = __all_sync(0xffffffffu, mbar_wait(bar(B_VFULL + s), (it >> 1) & 1, &abort_flag));
        if (!ok) { fail_id = B_VFULL + s + 1; break; }
        if constexpr (EARLY) {
          // next tile's QK^T as soon as this tile's S rows have been read
#pragma unroll
          for (int X = 0; X < 2; ++X) {
            if (!ok || it + 1 >= total_tiles) break;
            ok = __all_sync(0xffffffffu, mbar_wait(bar(B_SREAD + X), it & 1, &abort_flag));
            if (!ok) { fail_id = B_SREAD + X + 1; break; }
            tc_fence_after();
            ok = issue_qk(X, it + 1);
          }
        }
#pragma unroll
        for (int X = 0; X < 2; ++X) {
          if (!ok) break;
          if constexpr (!EARLY) {
            // first 64 keys of P V as soon as that half of P is written
            ok = __all_sync(0xffffffffu, mbar_wait_spin(bar(B_PHALF + X), it & 1, &abort_flag));
            if (!ok) { fail_id = B_PHALF + X + 1; break; }
            tc_fence_after();
            if (leader) {
              if (fresh) mma_ts(tOx[X], tPx[X], dV[s], IDESC_PV, 0u);
              else mma_ts(tOx[X], tPx[X], dV[s], IDESC_PV, 1u);
#pragma unroll
              for (int kk = 1; kk < 4; ++kk) mma_ts(tOx[X], tPx[X] + kk * 8, dV[s] + kk * 128, IDESC_PV, 1u);
            }
            __syncwarp();
          }
          ok = __all_sync(0xffffffffu, mbar_wait_spin(bar(B_PFULL + X), it & 1, &abort_flag));
          if (!ok) { fail_id = B_PFULL + X + 1; break; }
          tc_fence_after();
          if (leader) {
            if constexpr (EARLY) {
              if (fresh) mma_ts(tOx[X], tPx[X], dV[s], IDESC_PV, 0u);
              else mma_ts(tOx[X], tPx[X], dV[s], IDESC_PV, 1u);
#pragma unroll
              for (int kk = 1; kk < 4; ++kk) mma_ts(tOx[X], tPx[X] + kk * 8, dV[s] + kk * 128, IDESC_PV, 1u);
            }
            if (nch == 2) {
#pragma unroll
              for (int kk = 4; kk < 8; ++kk) mma_ts(tOx[X], tPx[X] + kk * 8, dV[s] + kk * 128, IDESC_PV, 1u);
            }
            tc_commit(bar(B_PVDONE + X));
            if (X == 1) tc_commit(bar(B_VEMPTY + s));
          }
          __syncwarp();
          if (!EARLY && it + 1 < total_tiles) ok = issue_qk(X, it + 1);
        }
        ++p_t; skip_empty(p_br, p_t);
        if (it + 1 < total_tiles) { ++q_t; skip_empty(q_br, q_t); }
      }
    }
  } else if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 72;\n");
    if constexpr (IN8) {
      // =============================== fp8 -> 16-bit converters ===============================
      // warp 2: K side (Q tile 0 first), warp 3: V side (Q tile 1 first).  A staged row of D fp8 bytes
      // becomes D values bf16(fp32(x) * scale) -- the operands the reference's wrapper builds
      // (nsa/triton/fp8.py:67-69), so the MMAs see exactly what the bf16 path sees on dequantised
      // tensors -- written in the 128-byte swizzled layout the MMA descriptors expect.
      const int side = warp - 2;
      const unsigned char* src = stg + side * STG;
      const __nv_fp8_interpretation_t kind = a.q_dtype == NSA_FP8_E5M2 ? __NV_E5M2 : __NV_E4M3;
      auto convert_rows = [&](int nrows, unsigned char* dst_tile, float dq) {
        constexpr int GPR = D / 16;                       // 16-element groups per row
        for (int i = lane; i < nrows * GPR; i += 32) {
          const int r = i / GPR, grp = i % GPR;
          const uint4 raw = *reinterpret_cast<const uint4*>(src + r * D + grp * 16);
          const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
          uint32_t o[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const __nv_fp8x2_storage_t two = (__nv_fp8x2_storage_t)((w[e >> 1] >> ((e & 1) * 16)) & 0xffffu);
            const __half2_raw h2 = __nv_cvt_fp8x2_to_halfraw2(two, kind);
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&h2));
            o[e] = Elem<__nv_bfloat16>::pack(f.x * dq, f.y * dq);
          }
          const int e0 = grp * 16, dh = e0 >> 6, ch = (e0 & 63) >> 3;        // two consecutive 16-byte chunks
          unsigned char* rowp = dst_tile + dh * DHSTRIDE + r * 128;
          *reinterpret_cast<uint4*>(rowp + (((ch) ^ (r & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
          *reinterpret_cast<uint4*>(rowp + (((ch + 1) ^ (r & 7)) << 4)) = make_uint4(o[4], o[5], o[6], o[7]);
        }
      };
      bool ok = __all_sync(0xffffffffu, mbar_wait(bar(B_STGFULL + side), 0, &abort_flag));
      if (!ok) fail_id = B_STGFULL + side + 1;
      if (ok) {
        convert_rows(128, smem + side * QTILE, a.q_scale);
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) { mbar_arrive(bar(B_QFULL)); mbar_arrive(bar(B_STGEMPTY + side)); }
      }
      int it = 0, u8 = 1;
      for (int br = 0; br < 3 && ok; ++br) {
        if (br == 0 || !p.kv8) { it += tend(br) - tbeg(br); continue; }   // 16-bit tiles come straight from TMA
        for (int t = tbeg(br); t < tend(br) && ok; ++t, ++it, ++u8) {
          const Tile tl = get_tile(br, t);
          const int s = it & 1, ph = (it >> 1) & 1;
          ok = __all_sync(0xffffffffu, mbar_wait(bar(B_STGFULL + side), u8 & 1, &abort_flag));
          if (!ok) { fail_id = B_STGFULL + side + 1; break; }
          ok = __all_sync(0xffffffffu, mbar_wait(bar((side == 0 ? B_KEMPTY : B_VEMPTY) + s), ph ^ 1, &abort_flag));
          if (!ok) { fail_id = (side == 0 ? B_KEMPTY : B_VEMPTY) + s + 1; break; }
          convert_rows(tl.nch * 64, smem + 2 * QTILE + (side == 0 ? 0 : 2 * KVTILE) + s * KVTILE, side == 0 ? a.k_scale : a.v_scale);
          fence_proxy_async();
          __syncwarp();
          if (lane == 0) { mbar_arrive(bar((side == 0 ? B_KFULL : B_VFULL) + s)); mbar_arrive(bar(B_STGEMPTY + side)); }
        }
      }
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 216;\n");
    // =============================== softmax / epilogue ===============================
    const int X = (warp - 4) >> 2;
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;                       // row of the tile == TMEM lane
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const uint32_t tS = tmem + lane_addr + X * 128;
    const uint32_t tO = tmem + lane_addr + 256 + X * 128;
    const uint32_t tP = EARLY ? tmem + lane_addr + 320 + X * 128 : tS;   // P: own columns at D=64, else over S
    const int rg = 2 * X + (r >> 6);                         // row group of this row
    const int head = grp_head(rg);
    const int qi = grp_qb(rg) * 64 + (r & 63);
    const bool row_ok = grp_qb(rg) < a.nq && qi < a.Tq;
    const size_t row_index = ((size_t)b * a.H + head) * a.Tq + qi;       // [B,H,Tq] order (lse, default out / gates)
    const size_t row_bthd = ((size_t)b * a.Tq + qi) * a.H + head;        // [B,Tq,H] order

    float gate[3] = {0.5f, 0.5f, 0.5f};
    if (a.fused) {
      float x[3] = {0.f, 0.f, 0.f};
      if (a.gates != nullptr && row_ok) {
#pragma unroll
        for (int c = 0; c < 3; ++c) {
          const size_t gi = ((a.io_layout & NSA_IO_GATES_BTHD) ? row_bthd : row_index) * 3 + c;
          x[c] = a.gate_dtype == NSA_FP32 ? reinterpret_cast<const float*>(a.gates)[gi]
               : a.gate_dtype == NSA_FP16 ? __half2float(reinterpret_cast<const __half*>(a.gates)[gi])
                                          : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(a.gates)[gi]);
        }
      }
      if (a.gate_act == NSA_GATE_SOFTMAX) {
        float mx = fmaxf(x[0], fmaxf(x[1], x[2]));
        float e0 = __expf(x[0] - mx), e1 = __expf(x[1] - mx), e2 = __expf(x[2] - mx);
        float inv = 1.f / (e0 + e1 + e2);
        gate[0] = e0 * inv; gate[1] = e1 * inv; gate[2] = e2 * inv;
      } else {
#pragma unroll
        for (int c = 0; c < 3; ++c) gate[c] = 1.f / (1.f + __expf(-x[c]));
      }
    }

    // The gated sum of the finished branches lives in the output row itself (16-bit, this thread's
    // own 2*D bytes of HBM, read back and added to at the next branch end): that keeps the whole
    // S row (128 registers) resident during a tile, so a tile costs ONE TMEM round trip.
    float lse_out = -INFINITY;
    bool have_partial = !SPLIT && a.accumulate != 0;       // the output row already holds a gated partial sum to add to
    T* orow = reinterpret_cast<T*>(a.out) + ((a.io_layout & NSA_IO_OUT_BTHD) ? row_bthd : row_index) * D;
    // Between branch ends the first 64 columns of the row's gated sum stay in shared memory (128 bytes per row, 16-byte
    // piece k at k ^ (row & 7): neighbouring rows on different banks) instead of going to the output row and back: a
    // thread reading or writing its own row in global memory touches 32 lines per instruction, and at D = 128 those
    // loads and stores were 12 % of the kernel.  Only the item's last branch writes these columns out; the values
    // are the same, rounded to 16 bits at every branch end.  At D = 64 that is the whole row.
    const bool keep = !SPLIT && !IN8 && p.psum != 0;
    unsigned char* prow_s = smem + 2 * QTILE + 4 * KVTILE + (size_t)(X * 128 + r) * 128;
    bool kept = false;                                   // the shared-memory columns hold a partial sum
    // The item's LAST branch end (every column goes to the output row) stages its 16-bit values in shared memory -- columns
    // 0..63 where the partial sums lay, 64..127 in the Q tiles' area, which no MMA reads any more -- as two boxes of 32 rows
    // x 128 bytes per warp (128-byte swizzle, the partial sums' own layout) and hands them to the TMA: the 16 stores per
    // thread, 32 lines each, were the longest part of an item's tail.  Rows past Tq are clipped by the tensor map.
    const bool fin_tma = keep && p.fin_tma != 0 && D == 128;
    unsigned char* fin_lo = smem + 2 * QTILE + 4 * KVTILE + (size_t)(warp - 4) * 4096;      // = this warp's rows of prow_s
    unsigned char* fin_hi = smem + (size_t)(warp - 4) * 4096;
    const int qi0_box = grp_qb(rg) * 64 + (quarter & 1) * 32;
    const bool box_ok = grp_qb(rg) < a.nq && qi0_box < a.Tq;
    int last_br = -1;                                    // the item's last branch with key tiles
#pragma unroll
    for (int br = 0; br < 3; ++br)
      if (tend(br) != tbeg(br)) last_br = br;

    int it = 0;
    bool ok = true;
#pragma unroll 1
    for (int br = 0; br < 3 && ok; ++br) {
      float* prow = nullptr;                                 // split launches: this row's partial result of the branch
      if constexpr (SPLIT) prow = p.part + ((row_index * p.nsplit + split) * 3 + br) * (D + 4);
      if (tend(br) == tbeg(br)) {
        if (SPLIT && row_ok) { prow[D] = -INFINITY; prow[D + 1] = 0.f; }
        continue;
      }
      int lo, hi;
      bounds(br, qi, row_ok, lo, hi);
      float m_used = -INFINITY, l = 0.f;
      const float sl2 = p.scale_log2[br];
#pragma unroll 1
      for (int t = tbeg(br); t < tend(br) && ok; ++t, ++it) {
        const Tile tl = get_tile(br, t);
        ok = __all_sync(0xffffffffu, mbar_wait(bar(B_SFULL + X), it & 1, &abort_flag));
        if (!ok) { fail_id = B_SFULL + X + 1; break; }
        tc_fence_after();
        // the whole S row of the tile: 64*nch columns, one wait
        uint32_t sv[4][32];
        tmem_ld32(tS, sv[0]);
        tmem_ld32(tS + 32, sv[1]);
        if (tl.nch == 2) { tmem_ld32(tS + 64, sv[2]); tmem_ld32(tS + 96, sv[3]); }
        tc_wait_ld();
        if constexpr (EARLY) {                             // S is in registers: the MMA warp may overwrite it
          tc_fence_before();
          mbar_arrive(bar(B_SREAD + X));
        }
        // valid column range of each chunk for this row; masked entries become -inf
        bool masked = false;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int vlo = max(lo - tl.j0[c], 0);
          const int vhi = (c < tl.nch && ((tl.mask[c] >> rg) & 1)) ? min(hi, tl.jlim[c] - 1) - tl.j0[c] : -1;
          if (c < tl.nch && (vlo > 0 || vhi < 63)) {
            masked = true;
#pragma unroll
            for (int g = 0; g < 2; ++g)
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (g * 32 + i < vlo || g * 32 + i > vhi) sv[2 * c + g][i] = 0xff800000u;   // -inf
          }
        }
        const bool use_poly = p.poly != 0 && !__any_sync(0xffffffffu, masked);
        float mx = row_max_raw(sv, tl.nch);
        mx *= p.scale_log2[br];                              // scale > 0 keeps the order
        // lazy rescale: only when some row of the warp outgrows its reference maximum by 2^8
        const bool grow = mx > m_used + 8.f;
        if (__any_sync(0xffffffffu, grow)) {
          const float m_new = fmaxf(m_used, mx);
          const float alpha = m_new == -INFINITY ? 1.f : ex2(m_used - m_new);
          if (t > tbeg(br)) {
            ok = __all_sync(0xffffffffu, mbar_wait(bar(B_PVDONE + X), (it - 1) & 1, &abort_flag));
            if (!ok) { fail_id = B_PVDONE + X + 1; break; }
            tc_fence_after();
            for (int g = 0; g < D / 32; ++g) {
              uint32_t v[32];
              tmem_ld32(tO + g * 32, v);
              tc_wait_ld();
#pragma unroll
              for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
              tmem_st32(tO + g * 32, v);
            }
            tc_wait_st();
          }
          l *= alpha;
          m_used = m_new;
        }
        const float m_ref = m_used == -INFINITY ? 0.f : m_used;
        if constexpr (EARLY) {
          if (it > 0) {                                    // P's columns are free once the previous PV has read them
            ok = __all_sync(0xffffffffu, mbar_wait(bar(B_PVDONE + X), (it - 1) & 1, &abort_flag));
            if (!ok) { fail_id = B_PVDONE + X + 1; break; }
            tc_fence_after();
          }
        }
        // P = exp2(S*scale - m_ref) as 16-bit (-inf -> 0)
        if (use_poly) {
          const f32x2 SL = mk2(sl2, sl2), NM = mk2(-m_ref, -m_ref);
          f32x2 sa = mk2(0.f, 0.f), sb = mk2(0.f, 0.f);
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            if (g < 2 * tl.nch) {
              uint32_t pk[16];
              exp_group_mixed<T>(sv[g], SL, NM, sa, sb, pk);
              tmem_st16(tP + g * 16, pk);
            }
            if (!EARLY && g == 1) { tc_wait_st(); tc_fence_before(); mbar_arrive(bar(B_PHALF + X)); }
          }
          float s0, s1;
          un2(add2(sa, sb), s0, s1);
          l += s0 + s1;
        } else {
          float psum0 = 0.f, psum1 = 0.f, psum2 = 0.f, psum3 = 0.f;
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            if (g < 2 * tl.nch) {
              uint32_t pk[16];
#pragma unroll
              for (int i = 0; i < 16; ++i) {
                const float p0 = ex2(fmaf(__uint_as_float(sv[g][2 * i]), sl2, -m_ref));
                const float p1 = ex2(fmaf(__uint_as_float(sv[g][2 * i + 1]), sl2, -m_ref));
                if (i & 1) { psum2 += p0; psum3 += p1; } else { psum0 += p0; psum1 += p1; }
                pk[i] = Elem<T>::pack(p0, p1);
              }
              tmem_st16(tP + g * 16, pk);
            }
            if (!EARLY && g == 1) { tc_wait_st(); tc_fence_before(); mbar_arrive(bar(B_PHALF + X)); }
          }
          psum0 += psum2;
          psum1 += psum3;
          l += psum0 + psum1;
        }
        tc_wait_st();
        tc_fence_before();
        mbar_arrive(bar(B_PFULL + X));
      }
      if (!ok) break;
      // ---- end of the branch: O is complete once the last PV has landed ---------------------------
      // The running gated sum of the earlier branches is read back from the output row NOW, before that wait: the
      // loads fly while the last PV executes instead of costing a memory round trip per 64 bytes afterwards.
      uint4 prevv[D / 8];
      if constexpr (!SPLIT) {
#pragma unroll
        for (int c = 0; c < D / 8; ++c) {
          if (c < 8 && kept) prevv[c] = *reinterpret_cast<const uint4*>(prow_s + ((c ^ (r & 7)) << 4));
          else prevv[c] = (have_partial && row_ok) ? reinterpret_cast<const uint4*>(orow)[c] : make_uint4(0u, 0u, 0u, 0u);
        }
      }
      ok = __all_sync(0xffffffffu, mbar_wait(bar(B_PVDONE + X), (it - 1) & 1, &abort_flag));
      if (!ok) { fail_id = B_PVDONE + X + 1; break; }
      tc_fence_after();
      if constexpr (SPLIT) {
        // unnormalised O of this block's share of the keys, with the row's reference maximum and sum
#pragma unroll
        for (int g = 0; g < D / 32; ++g) {
          uint32_t v[32];
          tmem_ld32(tO + g * 32, v);
          tc_wait_ld();
          if (row_ok) {
#pragma unroll
            for (int c = 0; c < 8; ++c)
              reinterpret_cast<uint4*>(prow)[g * 8 + c] = make_uint4(v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
          }
        }
        if (row_ok) { prow[D] = m_used; prow[D + 1] = l; }
        tc_fence_before();
        continue;
      }
      const bool has = l > 0.f;
      const float coef = has ? (a.fused ? gate[br] : 1.f) * p.out_scale[br] / l : 0.f;
      if (a.lse != nullptr) lse_out = has ? m_used * kLn2 + __logf(l) : -INFINITY;   // one branch per launch when lse is asked for
#pragma unroll
      for (int g = 0; g < D / 32; ++g) {
        uint32_t v[32];
        tmem_ld32(tO + g * 32, v);
        tc_wait_ld();
        if (row_ok) {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const uint4 prev = prevv[g * 4 + c];
            const uint32_t pw[4] = {prev.x, prev.y, prev.z, prev.w};
            uint32_t w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 acc = Elem<T>::unpack(pw[e]);
              w[e] = Elem<T>::pack(fmaf(__uint_as_float(v[8 * c + 2 * e]), coef, acc.x),
                                   fmaf(__uint_as_float(v[8 * c + 2 * e + 1]), coef, acc.y));
            }
            if (keep && br != last_br && g * 4 + c < 8)
              *reinterpret_cast<uint4*>(prow_s + (((g * 4 + c) ^ (r & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
            else if (fin_tma && br == last_br)
              *reinterpret_cast<uint4*>((g < 2 ? fin_lo : fin_hi) + lane * 128 + ((((g & 1) * 4 + c) ^ (lane & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
            else
              reinterpret_cast<uint4*>(orow)[g * 4 + c] = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
      if (fin_tma && br == last_br) {
        fence_proxy_async();
        __syncwarp();
        if (lane == 0 && box_ok) {
          const bool bthd = (a.io_layout & NSA_IO_OUT_BTHD) != 0;
          tma_store_4d(&p.tmOf, smem_u32(fin_lo), 0, bthd ? head : qi0_box, bthd ? qi0_box : head, b);
          tma_store_4d(&p.tmOf, smem_u32(fin_hi), 64, bthd ? head : qi0_box, bthd ? qi0_box : head, b);
          bulk_commit();
        }
      }
      have_partial = true;
      kept = keep && br != last_br;
      tc_fence_before();
    }
    if (fin_tma && lane == 0) bulk_wait_read<0>();       // the boxes have been read before the block's shared memory goes
    if (!SPLIT && ok && row_ok) {
      if (!have_partial) {                    // no branch had a visible key: the row is zero
#pragma unroll
        for (int c = 0; c < D / 8; ++c) reinterpret_cast<uint4*>(orow)[c] = make_uint4(0u, 0u, 0u, 0u);
      }
      if (a.lse != nullptr) a.lse[row_index] = lse_out;
    }
  }

  // ---- teardown (every path reaches it) -------------------------------------------------------
  if (fail_id != 0) atomicCAS(&g_tc5_status, 0, fail_id);
  tc_fence_before();
  __syncthreads();
  if (abort_flag && warp == 0 && lane == 0) {
    // let copies already in flight land (bounded) before the block's shared memory is handed back
    if (!IN8)
      for (int i = 0; i < 20000 && !mbar_try_wait(bar(B_QFULL), 0); ++i) __nanosleep(100);
    if (last_k_it >= 0)
      for (int i = 0; i < 20000 && !mbar_try_wait(bar(B_KFULL + (last_k_it & 1)), (last_k_it >> 1) & 1); ++i) __nanosleep(100);
    if (last_v_it >= 0)
      for (int i = 0; i < 20000 && !mbar_try_wait(bar(B_VFULL + (last_v_it & 1)), (last_v_it >> 1) & 1); ++i) __nanosleep(100);
    if (last_u8 >= 0)
      for (int side = 0; side < 2; ++side)
        for (int i = 0; i < 20000 && !mbar_try_wait(bar(B_STGFULL + side), last_u8 & 1); ++i) __nanosleep(100);
  }
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, 512); }
}

// ---------------------------------------------------------------- persistent variant
// The same arithmetic, one thread block per SM looping over work items (the items are ordered long rows first and dealt
// out in alternating directions, so every block gets a like mix).  What a one-item block pays per item
// -- barrier set-up, TMEM allocation, the list of selected blocks, the Q load and the first K tile before the first
// MMA, and an idle tensor pipe during the last epilogue -- is overlapped with the neighbouring items instead:
//   * warp 2 builds the NEXT item's block list into the other of two list buffers while the current item runs;
//   * warp 0 requests the next item's Q tiles as soon as the MMA warp has committed the current item's last Q K^T
//     (Q's shared memory is then free), and goes straight on to the next item's K/V tiles, ring permitting;
//   * warp 1 issues the next item's first Q K^T while the softmax warps are still in the current item's last epilogue
//     (its first P V is ordered behind that epilogue by the P-ready barrier, which the softmax warps reach only after it).
// All barrier phases come from running counters (tiles, items) instead of per-item ones.  bf16/fp16 storage, unsplit.
// Registers after setmaxnreg: 8 softmax warps x 216, the other four warps 72 each -- every warp runs the common teardown
// code, which is compiled once for all roles, so no role may shrink below what that code uses (a version that cut the
// idle warp to 24 registers hung a GPU run: the only unbounded wait in this kernel is a block-wide barrier that a
// misbehaving warp never reaches).  The .inc calls take 8*48 = 384 registers per lane and the .dec calls release
// 4*96 = 384: what the .inc calls take must have been released by the same block, or they block forever.
enum { PB_LISTFULL = B_COUNT, PB_LISTEMPTY = B_COUNT + 2, PB_QFREE = B_COUNT + 4, PB_COUNT = B_COUNT + 5 };

template <int D, int FMT>
__global__ void __launch_bounds__(384, 1) nsa_fwd_tc5_persist_kernel(const __grid_constant__ Tc5Params p, int n_items) {
  using T = typename std::conditional<FMT == 1, __nv_bfloat16, __half>::type;
  constexpr int DH = D / 64;
  constexpr int QTILE = DH * 128 * 128;
  constexpr int KVTILE = DH * 128 * 128;
  constexpr int DHSTRIDE = 128 * 128;
  constexpr bool EARLY = (D == 64);
  const nsa_fwd_args& a = p.a;

  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sQ = smem_u32(smem);
  const uint32_t sK = sQ + 2 * QTILE;
  const uint32_t sV = sK + 2 * KVTILE;
  __shared__ __align__(8) uint64_t bars[PB_COUNT];
  __shared__ int sel_list[2][T5_MAX_ENT];
  __shared__ unsigned char sel_mask[2][T5_MAX_ENT];
  __shared__ int sel_n[2];
  __shared__ int ent_blk[T5_MAX_ENT];              // scratch of the list builder
  __shared__ unsigned char ent_p[T5_MAX_ENT];
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_flag;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  auto bar = [&](int id) { return smem_u32(&bars[id]); };
  const int G = a.H / a.Hkv;
  const int GH = p.GH, NQB = 4 / p.GH;
  const int per_q = a.B * a.Hkv * p.HG;
  // The k-th item of this block.  Items are ordered long rows first; dealing them out in alternating directions (block
  // j takes the j-th of an even round and the j-th from the end of an odd one) keeps the blocks' totals level.
  auto item_of = [&](int k) { return k * (int)gridDim.x + ((k & 1) ? (int)gridDim.x - 1 - (int)blockIdx.x : (int)blockIdx.x); };

  // a work item's coordinates (see nsa_fwd_tc5_kernel) and, once its block list is there, its tile counts
  struct Item {
    int b, hk, h_base, qb_base, q_first, i_last, kv_slab;
    int nchunks[3], sld_c0;
  };
  auto bounds = [&](int br, int i, bool ok, int& lo, int& hi) {
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
  auto coords = [&](int item) {
    Item it;
    const int qbg = p.NQG - 1 - item / per_q;          // long rows first
    const int rem = item % per_q;
    it.b = rem / (a.Hkv * p.HG);
    it.hk = (rem / p.HG) % a.Hkv;
    const int hg = rem % p.HG;
    it.h_base = it.hk * G + hg * GH;
    it.qb_base = qbg * NQB;
    it.q_first = it.qb_base * 64;
    it.i_last = min((min(it.qb_base + NQB, a.nq)) * 64, a.Tq) - 1;
    it.kv_slab = it.b * a.Hkv + it.hk;
    it.nchunks[0] = it.nchunks[1] = it.nchunks[2] = 0;
    it.sld_c0 = 0;
    return it;
  };
  auto counts = [&](Item& it, int n_sel) {               // needs the item's block list (n_sel)
    int lo_f, hi_f, lo_l, hi_l;
    if (a.branches & NSA_BRANCH_COMPRESSED) {
      bounds(0, it.i_last, true, lo_l, hi_l);
      it.nchunks[0] = hi_l < 0 ? 0 : hi_l / 64 + 1;
    }
    if (a.branches & NSA_BRANCH_SELECTED) it.nchunks[1] = n_sel;
    if (a.branches & NSA_BRANCH_SLIDING) {
      bounds(2, it.q_first, true, lo_f, hi_f);
      bounds(2, it.i_last, true, lo_l, hi_l);
      if (hi_l >= lo_f) { it.sld_c0 = lo_f / 64; it.nchunks[2] = hi_l / 64 - it.sld_c0 + 1; }
    }
  };
  auto ntiles = [&](const Item& it, int br) { return (it.nchunks[br] + 1) >> 1; };
  auto get_tile = [&](const Item& it, int lp, int br, int t) {
    Tile tl;
    tl.nch = min(2, it.nchunks[br] - 2 * t);
    for (int c = 0; c < 2; ++c) {
      int ci = min(2 * t + c, it.nchunks[br] - 1);
      tl.mask[c] = 0xF;
      if (br == 0) { tl.j0[c] = ci * 64; tl.jlim[c] = a.Nc; }
      else if (br == 1) { int blk = sel_list[lp][ci]; tl.j0[c] = blk * 64; tl.jlim[c] = min(blk * 64 + 64, a.sel_key_limit); tl.mask[c] = sel_mask[lp][ci]; }
      else { tl.j0[c] = (it.sld_c0 + ci) * 64; tl.jlim[c] = a.Tk; }
    }
    return tl;
  };
  auto grp_head = [&](const Item& it, int g) { return it.h_base + g % GH; };
  auto grp_qb = [&](const Item& it, int g) { return it.qb_base + g / GH; };

  if (tid == 0) {
    abort_flag = 0;
    for (int i = 0; i < PB_COUNT; ++i) {
      int cnt = 1;
      if (i == B_PFULL || i == B_PFULL + 1 || i == B_SREAD || i == B_SREAD + 1 || i == B_PHALF || i == B_PHALF + 1) cnt = 128;
      if (i == PB_LISTEMPTY || i == PB_LISTEMPTY + 1) cnt = 10;     // producer, MMA issuer and the 8 softmax warps
      mbar_init(bar(i), cnt);
    }
    fence_barrier_init();
  }
  if (warp == 1) { tmem_alloc(smem_u32(&tmem_base_s), 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_s;

  int fail_id = 0;
  int last_k_it = -1, last_v_it = -1, q_loads = 0;   // producer: what has been issued (for the drain after an abort)

  if (warp == 0) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 72;\n");
    // =============================== TMA producer ===============================
    const bool leader = elect_one();
    if (leader) {
      tma_prefetch_desc(&p.tmQ); tma_prefetch_desc(&p.tmK); tma_prefetch_desc(&p.tmV);
      if (a.branches & NSA_BRANCH_COMPRESSED) { tma_prefetch_desc(&p.tmKc); tma_prefetch_desc(&p.tmVc); }
    }
    __syncwarp();
    int it = 0, k = 0;
    bool ok = true;
    for (int item = item_of(0); item < n_items && ok; item = item_of(++k)) {
      const int lp = k & 1;
      Item im = coords(item);
      ok = __all_sync(0xffffffffu, mbar_wait(bar(PB_LISTFULL + lp), (k >> 1) & 1, &abort_flag));
      if (!ok) { fail_id = PB_LISTFULL + lp + 1; break; }
      counts(im, sel_n[lp]);
      if (ntiles(im, 0) + ntiles(im, 1) + ntiles(im, 2) > 0) {     // an item without a tile needs no Q (and the MMA warp skips it)
        // Q's shared memory is free once the previous item's last Q K^T has been read by the tensor pipe
        if (q_loads > 0) {
          ok = __all_sync(0xffffffffu, mbar_wait(bar(PB_QFREE), (q_loads - 1) & 1, &abort_flag));
          if (!ok) { fail_id = PB_QFREE + 1; break; }
        }
        if (leader) {
          mbar_expect_tx(bar(B_QFULL), 2 * QTILE);
          for (int X = 0; X < 2; ++X)
            for (int hh = 0; hh < 2; ++hh)
              for (int dh = 0; dh < DH; ++dh)
                tma_load_3d(sQ + X * QTILE + dh * DHSTRIDE + hh * 8192, &p.tmQ, bar(B_QFULL), dh * 64, grp_qb(im, 2 * X + hh) * 64,
                            im.b * a.H + grp_head(im, 2 * X + hh));
        }
        ++q_loads;
      }
      for (int br = 0; br < 3 && ok; ++br) {
        const CUtensorMap* mk = br == 0 ? &p.tmKc : &p.tmK;
        const CUtensorMap* mv = br == 0 ? &p.tmVc : &p.tmV;
        for (int t = 0; t < ntiles(im, br) && ok; ++t, ++it) {
          const Tile tl = get_tile(im, lp, br, t);
          const int s = it & 1, ph = (it >> 1) & 1;
          const uint32_t bytes = (uint32_t)tl.nch * 64 * D * 2;
          ok = __all_sync(0xffffffffu, mbar_wait(bar(B_KEMPTY + s), ph ^ 1, &abort_flag));
          if (!ok) { fail_id = B_KEMPTY + s + 1; break; }
          if (leader) {
            mbar_expect_tx(bar(B_KFULL + s), bytes);
            for (int c = 0; c < tl.nch; ++c)
              for (int dh = 0; dh < DH; ++dh)
                tma_load_3d(sK + s * KVTILE + dh * DHSTRIDE + c * 8192, mk, bar(B_KFULL + s), dh * 64, tl.j0[c], im.kv_slab);
          }
          last_k_it = it;
          ok = __all_sync(0xffffffffu, mbar_wait(bar(B_VEMPTY + s), ph ^ 1, &abort_flag));
          if (!ok) { fail_id = B_VEMPTY + s + 1; break; }
          if (leader) {
            mbar_expect_tx(bar(B_VFULL + s), bytes);
            for (int c = 0; c < tl.nch; ++c)
              for (int dh = 0; dh < DH; ++dh)
                tma_load_3d(sV + s * KVTILE + dh * DHSTRIDE + c * 8192, mv, bar(B_VFULL + s), dh * 64, tl.j0[c], im.kv_slab);
          }
          last_v_it = it;
          __syncwarp();
        }
      }
      if (ok && lane == 0) mbar_arrive(bar(PB_LISTEMPTY + lp));
      __syncwarp();
    }
  } else if (warp == 1) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 72;\n");
    // =============================== MMA issuer ===============================
    const bool leader = elect_one();
    constexpr uint32_t IDESC_PV = idesc_f16(FMT, 128, D, 0, 1);
    constexpr uint32_t IDESC_QK1 = idesc_f16(FMT, 128, 64, 0, 0);
    constexpr uint32_t IDESC_QK2 = idesc_f16(FMT, 128, 128, 0, 0);
    const uint64_t dQ[2] = {smem_desc_sw128(sQ, 16, 1024), smem_desc_sw128(sQ + QTILE, 16, 1024)};
    const uint64_t dK[2] = {smem_desc_sw128(sK, 16, 1024), smem_desc_sw128(sK + KVTILE, 16, 1024)};
    const uint64_t dV[2] = {smem_desc_sw128(sV, DHSTRIDE, 1024), smem_desc_sw128(sV + KVTILE, DHSTRIDE, 1024)};
    const uint32_t tSx[2] = {tmem, tmem + 128}, tOx[2] = {tmem + 256, tmem + 384};
    const uint32_t tPx[2] = {EARLY ? tmem + 320 : tmem, EARLY ? tmem + 448 : tmem + 128};
    bool ok = true;

    // The issuer walks two cursors over the flattened (item, branch, tile) sequence: q = the tile whose Q K^T is
    // issued next, v = the tile whose P V is issued next; q is one tile ahead of v and crosses into the next item
    // first.  Items without a tile are skipped (nothing is loaded or issued for them).
    // (scalars only: the cursors are read between every two MMA issues, and an array indexed by the branch would put them
    // in local memory)
    struct Cur { int item, k, f, ntot, it, live, c0, c1, c2, n0, n01; bool valid; };
    auto open_item = [&](Cur& c, int item, int kk) -> bool {      // positions c on the first tile of `item` or of the next item that has one
      c.item = item; c.k = kk; c.valid = false;
      while (c.item < n_items) {
        const int lp = c.k & 1;
        if (!__all_sync(0xffffffffu, mbar_wait(bar(PB_LISTFULL + lp), (c.k >> 1) & 1, &abort_flag))) { fail_id = PB_LISTFULL + lp + 1; return false; }
        Item im = coords(c.item);
        counts(im, sel_n[lp]);
        c.c0 = im.nchunks[0]; c.c1 = im.nchunks[1]; c.c2 = im.nchunks[2];
        c.n0 = (c.c0 + 1) >> 1;
        c.n01 = c.n0 + ((c.c1 + 1) >> 1);
        c.ntot = c.n01 + ((c.c2 + 1) >> 1);
        c.f = 0;
        if (c.ntot > 0) { c.valid = true; ++c.live; return true; }
        ++c.k; c.item = item_of(c.k);
      }
      return true;
    };
    auto advance = [&](Cur& c) -> bool {                           // next tile; crosses item boundaries
      ++c.f; ++c.it;
      if (c.f < c.ntot) return true;
      return open_item(c, item_of(c.k + 1), c.k + 1);
    };
    // chunks (1 or 2) of the cursor's tile, and whether it opens a branch
    auto tile_of = [](const Cur& c, int& nch, bool& fresh) {
      int t, cb;
      if (c.f < c.n0) { t = c.f; cb = c.c0; }
      else if (c.f < c.n01) { t = c.f - c.n0; cb = c.c1; }
      else { t = c.f - c.n01; cb = c.c2; }
      nch = min(2, cb - 2 * t);
      fresh = t == 0;
    };
    auto release_lists = [&](int k0, int k1) {                     // this warp is done with the block lists of items k0..k1-1
      for (int kk = k0; kk < k1; ++kk)
        if (lane == 0) mbar_arrive(bar(PB_LISTEMPTY + (kk & 1)));
      __syncwarp();
    };
    Cur q;
    q.it = 0; q.live = 0;
    ok = open_item(q, item_of(0), 0);
    Cur v = q;
    if (ok) release_lists(0, v.k);                                 // leading items without a tile
    int q_ready = 0;                  // live items whose Q is known to have landed

    auto issue_qk = [&](int X) -> bool {     // Q K^T of tile q for 128-row tile X
      const int s = q.it & 1;
      if (X == 0) {
        if (q.live > q_ready) {              // first tile of an item: its Q must be in shared memory
          if (!__all_sync(0xffffffffu, mbar_wait(bar(B_QFULL), (q.live - 1) & 1, &abort_flag))) { fail_id = B_QFULL + 1; return false; }
          q_ready = q.live;
        }
        if (!__all_sync(0xffffffffu, mbar_wait(bar(B_KFULL + s), (q.it >> 1) & 1, &abort_flag))) { fail_id = B_KFULL + s + 1; return false; }
        tc_fence_after();
      }
      int nch; bool fr;
      tile_of(q, nch, fr);
      const uint32_t idesc = nch == 2 ? IDESC_QK2 : IDESC_QK1;
      const bool last = X == 1 && q.f == q.ntot - 1;   // the item's last tile: its Q is free once these MMAs have read it
      if (leader) {
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const uint32_t off = (uint32_t)(((ks >> 2) * DHSTRIDE + (ks & 3) * 32) >> 4);
          if (ks == 0) mma_ss(tSx[X], dQ[X] + off, dK[s] + off, idesc, 0u);
          else mma_ss(tSx[X], dQ[X] + off, dK[s] + off, idesc, 1u);
        }
        tc_commit(bar(B_SFULL + X));
        if (X == 1) tc_commit(bar(B_KEMPTY + s));
        if (last) tc_commit(bar(PB_QFREE));
      }
      __syncwarp();
      return true;
    };

    if (ok && q.valid) {
      ok = issue_qk(0) && issue_qk(1);
      if (ok) ok = advance(q);
    }
    while (ok && v.valid) {
      const int it = v.it;
      int nch; bool fresh;                               // fresh: first tile of a branch starts a new O
      tile_of(v, nch, fresh);
      const int s = it & 1;
      // Q K^T of the next tile is interleaved with this tile's P V -- unless it belongs to the next item: its Q arrives a
      // TMA round trip after this item's last Q K^T, and waiting for it here would hold up this item's last P V
      const bool same_item = q.valid && q.k == v.k;
      ok = __all_sync(0xffffffffu, mbar_wait(bar(B_VFULL + s), (it >> 1) & 1, &abort_flag));
      if (!ok) { fail_id = B_VFULL + s + 1; break; }
      if constexpr (EARLY) {
#pragma unroll
        for (int X = 0; X < 2; ++X) {
          if (!ok || !same_item) break;
          ok = __all_sync(0xffffffffu, mbar_wait(bar(B_SREAD + X), it & 1, &abort_flag));
          if (!ok) { fail_id = B_SREAD + X + 1; break; }
          tc_fence_after();
          ok = issue_qk(X);
        }
      }
#pragma unroll
      for (int X = 0; X < 2; ++X) {
        if (!ok) break;
        ok = __all_sync(0xffffffffu, mbar_wait(bar(B_PFULL + X), it & 1, &abort_flag));
        if (!ok) { fail_id = B_PFULL + X + 1; break; }
        tc_fence_after();
        if (leader) {
          if (fresh) mma_ts(tOx[X], tPx[X], dV[s], IDESC_PV, 0u);
          else mma_ts(tOx[X], tPx[X], dV[s], IDESC_PV, 1u);
#pragma unroll
          for (int kk = 1; kk < 4; ++kk) mma_ts(tOx[X], tPx[X] + kk * 8, dV[s] + kk * 128, IDESC_PV, 1u);
          if (nch == 2) {
#pragma unroll
            for (int kk = 4; kk < 8; ++kk) mma_ts(tOx[X], tPx[X] + kk * 8, dV[s] + kk * 128, IDESC_PV, 1u);
          }
          tc_commit(bar(B_PVDONE + X));
          if (X == 1) tc_commit(bar(B_VEMPTY + s));
        }
        __syncwarp();
        if (!EARLY && same_item) ok = issue_qk(X);
      }
      if (!ok) break;
      if (q.valid && !same_item) {
        // first tile of the next item, behind this item's last P V (S aliases P at D=128; at D=64 the S rows of this
        // item's last tile have been read long before its P was written)
        ok = issue_qk(0) && issue_qk(1);
        if (!ok) break;
      }
      // v first: leaving an item releases its block list, which the builder may need before it can build the list q is
      // about to ask for (an item of a single tile puts q two items ahead of the list v still holds)
      const int k_before = v.k;
      ok = advance(v);
      if (ok && v.k != k_before) release_lists(k_before, v.k);
      if (ok && q.valid) ok = advance(q);
    }
  } else if (warp == 2) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 72;\n");
    // =============================== block-list builder ===============================
    int k = 0;
    bool ok = true;
    for (int item = item_of(0); item < n_items && ok; item = item_of(++k)) {
      const int lp = k & 1;
      const Item im = coords(item);
      ok = __all_sync(0xffffffffu, mbar_wait(bar(PB_LISTEMPTY + lp), ((k >> 1) & 1) ^ 1, &abort_flag));
      if (!ok) { fail_id = PB_LISTEMPTY + lp + 1; break; }
      int n = 0;
      if (a.branches & NSA_BRANCH_SELECTED) {
        const bool shared = a.Hi != a.H && GH == 4;
        const int ngrp = shared ? 1 : 4;
        const int n_ent = ngrp * a.top_k;
        for (int i = lane; i < n_ent; i += 32) {
          const int g = i / a.top_k, sl = i % a.top_k;
          const int qb = grp_qb(im, g);
          int blk = -1;
          if (qb < a.nq) {
            const int hi_ = (a.Hi == a.H) ? grp_head(im, g) : im.hk;
            blk = a.idx[(((size_t)im.b * a.Hi + hi_) * a.nq + qb) * a.top_k + sl];
            const int last_pos = min(qb * 64 + 64, a.Tq) - 1 + a.offset;
            if (blk < 0 || blk >= a.sel_key_limit / 64 || (a.causal && (long long)blk * 64 > last_pos)) blk = -1;
          }
          ent_blk[i] = blk;
        }
        __syncwarp();
        if (!shared) {
          for (int i = lane; i < n_ent; i += 32) {
            int pc = 0;
            const int blk = ent_blk[i], g0 = (i / a.top_k) * a.top_k;
            for (int j = g0; j < i; ++j) pc += (ent_blk[j] == blk);
            ent_p[i] = (unsigned char)pc;
          }
          __syncwarp();
        }
        for (int i0 = 0; i0 < n_ent; i0 += 32) {
          const int i = i0 + lane;
          bool lead = false;
          unsigned msk = 0xFu;
          if (i < n_ent && ent_blk[i] >= 0) {
            lead = true;
            if (!shared) {
              const int blk = ent_blk[i], pi = ent_p[i], gi = i / a.top_k;
              msk = 0;
              for (int j = 0; j < n_ent; ++j) {
                if (ent_blk[j] == blk && ent_p[j] == pi) {
                  const int gj = j / a.top_k;
                  msk |= 1u << gj;
                  if (gj < gi) lead = false;
                }
              }
            }
          }
          const unsigned bal = __ballot_sync(0xffffffffu, lead);
          if (lead) {
            const int pos = n + __popc(bal & ((1u << lane) - 1));
            sel_list[lp][pos] = ent_blk[i];
            sel_mask[lp][pos] = (unsigned char)msk;
          }
          n += __popc(bal);
        }
      }
      if (lane == 0) sel_n[lp] = n;
      __syncwarp();
      __threadfence_block();
      if (lane == 0) mbar_arrive(bar(PB_LISTFULL + lp));
      __syncwarp();
    }
  } else if (warp == 3) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 72;\n");
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 216;\n");
    // =============================== softmax / epilogue ===============================
    const int X = (warp - 4) >> 2;
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const uint32_t tS = tmem + lane_addr + X * 128;
    const uint32_t tO = tmem + lane_addr + 256 + X * 128;
    const uint32_t tP = EARLY ? tmem + lane_addr + 320 + X * 128 : tS;
    const int rg = 2 * X + (r >> 6);
    int it = 0, k = 0;
    bool ok = true;
#pragma unroll 1
    for (int item = item_of(0); item < n_items && ok; item = item_of(++k)) {
      const int lp = k & 1;
      Item im = coords(item);
      const int head = grp_head(im, rg);
      const int qi = grp_qb(im, rg) * 64 + (r & 63);
      const bool row_ok = grp_qb(im, rg) < a.nq && qi < a.Tq;
      const size_t row_index = ((size_t)im.b * a.H + head) * a.Tq + qi;
      const size_t row_bthd = ((size_t)im.b * a.Tq + qi) * a.H + head;
      // gate logits: the loads are issued here and first touched at a branch end, long after they have arrived
      float gx[3] = {0.f, 0.f, 0.f};
      if (a.fused && a.gates != nullptr && row_ok) {
#pragma unroll
        for (int c = 0; c < 3; ++c) {
          const size_t gi = ((a.io_layout & NSA_IO_GATES_BTHD) ? row_bthd : row_index) * 3 + c;
          gx[c] = a.gate_dtype == NSA_FP32 ? reinterpret_cast<const float*>(a.gates)[gi]
                : a.gate_dtype == NSA_FP16 ? __half2float(reinterpret_cast<const __half*>(a.gates)[gi])
                                           : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(a.gates)[gi]);
        }
      }
      auto gate_of = [&](int br) {
        if (a.gate_act == NSA_GATE_SOFTMAX) {
          const float mx = fmaxf(gx[0], fmaxf(gx[1], gx[2]));
          const float e0 = __expf(gx[0] - mx), e1 = __expf(gx[1] - mx), e2 = __expf(gx[2] - mx);
          return (br == 0 ? e0 : br == 1 ? e1 : e2) / (e0 + e1 + e2);
        }
        const float x = br == 0 ? gx[0] : br == 1 ? gx[1] : gx[2];
        return 1.f / (1.f + __expf(-x));
      };
      float lse_out = -INFINITY;
      bool have_partial = a.accumulate != 0;
      T* orow = reinterpret_cast<T*>(a.out) + ((a.io_layout & NSA_IO_OUT_BTHD) ? row_bthd : row_index) * D;
      unsigned char* ostage = smem + 2 * QTILE + 4 * KVTILE + (warp - 4) * 2048;
      const int qi0_box = grp_qb(im, rg) * 64 + (quarter & 1) * 32;        // this warp's rows: 32 consecutive positions of one head
      const bool box_ok = grp_qb(im, rg) < a.nq && qi0_box < a.Tq;

      ok = __all_sync(0xffffffffu, mbar_wait(bar(PB_LISTFULL + lp), (k >> 1) & 1, &abort_flag));
      if (!ok) { fail_id = PB_LISTFULL + lp + 1; break; }
      counts(im, sel_n[lp]);
      const int n_with_tiles = (ntiles(im, 0) != 0) + (ntiles(im, 1) != 0) + (ntiles(im, 2) != 0);
#pragma unroll 1
      for (int br = 0; br < 3 && ok; ++br) {
        if (ntiles(im, br) == 0) continue;
        int lo, hi;
        bounds(br, qi, row_ok, lo, hi);
        float m_used = -INFINITY, l = 0.f;
        const float sl2 = p.scale_log2[br];
#pragma unroll 1
        for (int t = 0; t < ntiles(im, br) && ok; ++t, ++it) {
          const Tile tl = get_tile(im, lp, br, t);
          ok = __all_sync(0xffffffffu, mbar_wait(bar(B_SFULL + X), it & 1, &abort_flag));
          if (!ok) { fail_id = B_SFULL + X + 1; break; }
          tc_fence_after();
          uint32_t sv[4][32];
          tmem_ld32(tS, sv[0]);
          tmem_ld32(tS + 32, sv[1]);
          if (tl.nch == 2) { tmem_ld32(tS + 64, sv[2]); tmem_ld32(tS + 96, sv[3]); }
          tc_wait_ld();
          if constexpr (EARLY) {
            tc_fence_before();
            mbar_arrive(bar(B_SREAD + X));
          }
          bool masked = false;
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            const int vlo = max(lo - tl.j0[c], 0);
            const int vhi = (c < tl.nch && ((tl.mask[c] >> rg) & 1)) ? min(hi, tl.jlim[c] - 1) - tl.j0[c] : -1;
            if (c < tl.nch && (vlo > 0 || vhi < 63)) {
              masked = true;
#pragma unroll
              for (int g = 0; g < 2; ++g)
#pragma unroll
                for (int i = 0; i < 32; ++i)
                  if (g * 32 + i < vlo || g * 32 + i > vhi) sv[2 * c + g][i] = 0xff800000u;
            }
          }
          const bool use_poly = p.poly != 0 && !__any_sync(0xffffffffu, masked);
          float mx = row_max_raw(sv, tl.nch);
          mx *= p.scale_log2[br];
          const bool grow = mx > m_used + 8.f;
          if (__any_sync(0xffffffffu, grow)) {
            const float m_new = fmaxf(m_used, mx);
            const float alpha = m_new == -INFINITY ? 1.f : ex2(m_used - m_new);
            if (t > 0) {
              ok = __all_sync(0xffffffffu, mbar_wait(bar(B_PVDONE + X), (it - 1) & 1, &abort_flag));
              if (!ok) { fail_id = B_PVDONE + X + 1; break; }
              tc_fence_after();
              for (int g = 0; g < D / 32; ++g) {
                uint32_t v[32];
                tmem_ld32(tO + g * 32, v);
                tc_wait_ld();
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
                tmem_st32(tO + g * 32, v);
              }
              tc_wait_st();
            }
            l *= alpha;
            m_used = m_new;
          }
          const float m_ref = m_used == -INFINITY ? 0.f : m_used;
          if constexpr (EARLY) {
            if (it > 0) {
              ok = __all_sync(0xffffffffu, mbar_wait(bar(B_PVDONE + X), (it - 1) & 1, &abort_flag));
              if (!ok) { fail_id = B_PVDONE + X + 1; break; }
              tc_fence_after();
            }
          }
          if (use_poly) {
            const f32x2 SL = mk2(sl2, sl2), NM = mk2(-m_ref, -m_ref);
            f32x2 sa = mk2(0.f, 0.f), sb = mk2(0.f, 0.f);
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              if (g < 2 * tl.nch) {
                uint32_t pk[16];
                exp_group_mixed<T>(sv[g], SL, NM, sa, sb, pk);
                tmem_st16(tP + g * 16, pk);
              }
            }
            float s0, s1;
            un2(add2(sa, sb), s0, s1);
            l += s0 + s1;
          } else {
            float psum0 = 0.f, psum1 = 0.f, psum2 = 0.f, psum3 = 0.f;
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              if (g < 2 * tl.nch) {
                uint32_t pk[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                  const float p0 = ex2(fmaf(__uint_as_float(sv[g][2 * i]), sl2, -m_ref));
                  const float p1 = ex2(fmaf(__uint_as_float(sv[g][2 * i + 1]), sl2, -m_ref));
                  if (i & 1) { psum2 += p0; psum3 += p1; } else { psum0 += p0; psum1 += p1; }
                  pk[i] = Elem<T>::pack(p0, p1);
                }
                tmem_st16(tP + g * 16, pk);
              }
            }
            psum0 += psum2;
            psum1 += psum3;
            l += psum0 + psum1;
          }
          tc_wait_st();
          tc_fence_before();
          mbar_arrive(bar(B_PFULL + X));
        }
        if (!ok) break;
        // ---- end of the branch ----
        if (p.tma_out != 0 && n_with_tiles == 1 && !have_partial) {      // this branch alone is the item's result
          ok = __all_sync(0xffffffffu, mbar_wait(bar(B_PVDONE + X), (it - 1) & 1, &abort_flag));
          if (!ok) { fail_id = B_PVDONE + X + 1; break; }
          tc_fence_after();
          const bool has = l > 0.f;
          const float coef = has ? (a.fused ? gate_of(br) : 1.f) * p.out_scale[br] / l : 0.f;
          if (a.lse != nullptr) lse_out = has ? m_used * kLn2 + __logf(l) : -INFINITY;
          const bool bthd = (a.io_layout & NSA_IO_OUT_BTHD) != 0;
          if (box_ok)
            rows_through_tma<T, D>(ostage, tO, coef, lane, [&](uint32_t src, int col) {
              tma_store_4d(&p.tmO, src, col, bthd ? head : qi0_box, bthd ? qi0_box : head, im.b); });
          have_partial = true;
          tc_fence_before();
          continue;
        }
        uint4 prevv[D / 8];
#pragma unroll
        for (int c = 0; c < D / 8; ++c)
          prevv[c] = (have_partial && row_ok) ? reinterpret_cast<const uint4*>(orow)[c] : make_uint4(0u, 0u, 0u, 0u);
        ok = __all_sync(0xffffffffu, mbar_wait(bar(B_PVDONE + X), (it - 1) & 1, &abort_flag));
        if (!ok) { fail_id = B_PVDONE + X + 1; break; }
        tc_fence_after();
        const bool has = l > 0.f;
        const float coef = has ? (a.fused ? gate_of(br) : 1.f) * p.out_scale[br] / l : 0.f;
        if (a.lse != nullptr) lse_out = has ? m_used * kLn2 + __logf(l) : -INFINITY;
#pragma unroll
        for (int g = 0; g < D / 32; ++g) {
          uint32_t v[32];
          tmem_ld32(tO + g * 32, v);
          tc_wait_ld();
          if (row_ok) {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              const uint4 prev = prevv[g * 4 + c];
              const uint32_t pw[4] = {prev.x, prev.y, prev.z, prev.w};
              uint32_t w[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float2 acc = Elem<T>::unpack(pw[e]);
                w[e] = Elem<T>::pack(fmaf(__uint_as_float(v[8 * c + 2 * e]), coef, acc.x),
                                     fmaf(__uint_as_float(v[8 * c + 2 * e + 1]), coef, acc.y));
              }
              reinterpret_cast<uint4*>(orow)[g * 4 + c] = make_uint4(w[0], w[1], w[2], w[3]);
            }
          }
        }
        have_partial = true;
        tc_fence_before();
      }
      if (!ok) break;
      if (row_ok) {
        if (!have_partial) {
#pragma unroll
          for (int c = 0; c < D / 8; ++c) reinterpret_cast<uint4*>(orow)[c] = make_uint4(0u, 0u, 0u, 0u);
        }
        if (a.lse != nullptr) a.lse[row_index] = lse_out;
      }
      if (lane == 0) mbar_arrive(bar(PB_LISTEMPTY + lp));      // this warp is done with the item's block list
      __syncwarp();
    }
    if (p.tma_out != 0 && lane == 0) bulk_wait_read<0>();      // the staging area has been read before the block's shared memory goes
  }

  // ---- teardown ----
  if (fail_id != 0) atomicCAS(&g_tc5_status, 0, fail_id);
  tc_fence_before();
  __syncthreads();
  if (abort_flag && warp == 0 && lane == 0) {
    if (q_loads > 0)
      for (int i = 0; i < 20000 && !mbar_try_wait(bar(B_QFULL), (q_loads - 1) & 1); ++i) __nanosleep(100);
    if (last_k_it >= 0)
      for (int i = 0; i < 20000 && !mbar_try_wait(bar(B_KFULL + (last_k_it & 1)), (last_k_it >> 1) & 1); ++i) __nanosleep(100);
    if (last_v_it >= 0)
      for (int i = 0; i < 20000 && !mbar_try_wait(bar(B_VFULL + (last_v_it & 1)), (last_v_it >> 1) & 1); ++i) __nanosleep(100);
  }
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, 512); }
}

// Merges the partial results of a split launch: per row and branch, the splits' (O_s, m_s, l_s) combine to
// O = sum_s 2^(m_s - m) O_s / sum_s 2^(m_s - m) l_s with m = max_s m_s; the three branches are then added with
// the row's gates, in fp32, and the row is rounded once.  One warp per row, D/32 columns per lane.
template <typename T, int D>
__global__ void __launch_bounds__(256) nsa_split_combine_kernel(const float* __restrict__ part, T* __restrict__ out,
                                                                const void* __restrict__ gates, int gate_dtype, int gate_act,
                                                                int io_layout, int H, int Tq, long long rows, int nsplit,
                                                                float os0, float os1, float os2) {
  constexpr int CPT = D / 32;
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);     // (b, h, t) order
  if (row >= rows) return;
  const long long bh = row / Tq;
  const int t = (int)(row % Tq), h = (int)(bh % H);
  const long long b = bh / H;
  const long long row_bthd = (b * Tq + t) * H + h;
  float gate[3] = {0.5f, 0.5f, 0.5f};
  {
    float x[3] = {0.f, 0.f, 0.f};
    if (gates != nullptr) {
      const size_t gi = (size_t)((io_layout & NSA_IO_GATES_BTHD) ? row_bthd : row) * 3;
#pragma unroll
      for (int c = 0; c < 3; ++c)
        x[c] = gate_dtype == NSA_FP32 ? reinterpret_cast<const float*>(gates)[gi + c]
             : gate_dtype == NSA_FP16 ? __half2float(reinterpret_cast<const __half*>(gates)[gi + c])
                                      : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(gates)[gi + c]);
    }
    if (gate_act == NSA_GATE_SOFTMAX) {
      const float mx = fmaxf(x[0], fmaxf(x[1], x[2]));
      const float e0 = __expf(x[0] - mx), e1 = __expf(x[1] - mx), e2 = __expf(x[2] - mx);
      const float inv = 1.f / (e0 + e1 + e2);
      gate[0] = e0 * inv; gate[1] = e1 * inv; gate[2] = e2 * inv;
    } else {
#pragma unroll
      for (int c = 0; c < 3; ++c) gate[c] = 1.f / (1.f + __expf(-x[c]));
    }
  }
  const float os[3] = {os0, os1, os2};
  float acc[CPT];
#pragma unroll
  for (int c = 0; c < CPT; ++c) acc[c] = 0.f;
  const float* prow = part + (size_t)row * nsplit * 3 * (D + 4);
  constexpr int MAXS = 16;                                  // nsplit <= 16: every load of a step is issued before any is used
#pragma unroll
  for (int br = 0; br < 3; ++br) {
    float ms[MAXS], ls[MAXS];
#pragma unroll
    for (int s = 0; s < MAXS; ++s) {
      const bool in = s < nsplit;
      const float2 ml = in ? *reinterpret_cast<const float2*>(prow + (s * 3 + br) * (D + 4) + D) : make_float2(-INFINITY, 0.f);
      ms[s] = ml.x; ls[s] = ml.y;
    }
    float m = -INFINITY;
#pragma unroll
    for (int s = 0; s < MAXS; ++s) m = fmaxf(m, ms[s]);
    if (m == -INFINITY) continue;
    float l = 0.f, o[CPT];
#pragma unroll
    for (int c = 0; c < CPT; ++c) o[c] = 0.f;
#pragma unroll
    for (int s0 = 0; s0 < MAXS; s0 += 8) {
      if (s0 >= nsplit) break;
      float v[8][CPT];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const bool in = s0 + e < nsplit && ms[s0 + e] != -INFINITY;
        const float* ps = prow + ((s0 + e) * 3 + br) * (D + 4) + lane * CPT;
#pragma unroll
        for (int c = 0; c < CPT; ++c) v[e][c] = in ? ps[c] : 0.f;
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        if (s0 + e < nsplit && ms[s0 + e] != -INFINITY) {
          const float w = exp2f(ms[s0 + e] - m);
          l = fmaf(ls[s0 + e], w, l);
#pragma unroll
          for (int c = 0; c < CPT; ++c) o[c] = fmaf(v[e][c], w, o[c]);
        }
      }
    }
    if (l > 0.f) {
      const float coef = gate[br] * os[br] / l;
#pragma unroll
      for (int c = 0; c < CPT; ++c) acc[c] = fmaf(o[c], coef, acc[c]);
    }
  }
  T* orow = out + (size_t)((io_layout & NSA_IO_OUT_BTHD) ? row_bthd : row) * D + lane * CPT;
  if constexpr (CPT == 4) {
    *reinterpret_cast<uint2*>(orow) = make_uint2(Elem<T>::pack(acc[0], acc[1]), Elem<T>::pack(acc[2], acc[3]));
  } else {
    *reinterpret_cast<uint32_t*>(orow) = Elem<T>::pack(acc[0], acc[1]);
  }
}

// ---------------------------------------------------------------- host side
static PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  if (!fn) {
    cudaDriverEntryPointQueryResult q;
    void* ptr = nullptr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(ptr);
  }
  return fn;
}

// [slabs][rows][D] fp8 tensor, boxes of 64 rows x D bytes, no swizzle (the converter warps re-lay it out)
static int make_map8(CUtensorMap* m, const void* ptr, long long slabs, long long rows, int D) {
  auto enc = encode_fn();
  NSA_REQUIRE(enc != nullptr, NSA_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  NSA_REQUIRE((reinterpret_cast<uintptr_t>(ptr) & 15) == 0, NSA_ERR_ARG, "tensor base %p is not 16-byte aligned", ptr);
  cuuint64_t dims[3] = {(cuuint64_t)D, (cuuint64_t)rows, (cuuint64_t)slabs};
  cuuint64_t strides[2] = {(cuuint64_t)D, (cuuint64_t)rows * D};
  cuuint32_t box[3] = {(cuuint32_t)D, 64, 1};
  cuuint32_t es[3] = {1, 1, 1};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(ptr), dims, strides, box, es,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  NSA_REQUIRE(r == CUDA_SUCCESS, NSA_ERR_CUDA, "cuTensorMapEncodeTiled (fp8) failed with %d", (int)r);
  return NSA_OK;
}

// [slabs][rows][D] 16-bit tensor, boxes of 64 rows x 64 elements, 128-byte swizzle, zero fill outside
int make_map(CUtensorMap* m, const void* ptr, long long slabs, long long rows, int D, int dtype) {
  auto enc = encode_fn();
  NSA_REQUIRE(enc != nullptr, NSA_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  NSA_REQUIRE((reinterpret_cast<uintptr_t>(ptr) & 15) == 0, NSA_ERR_ARG, "tensor base %p is not 16-byte aligned", ptr);
  cuuint64_t dims[3] = {(cuuint64_t)D, (cuuint64_t)rows, (cuuint64_t)slabs};
  cuuint64_t strides[2] = {(cuuint64_t)D * 2, (cuuint64_t)rows * D * 2};
  cuuint32_t box[3] = {64, 64, 1};
  cuuint32_t es[3] = {1, 1, 1};
  CUresult r = enc(m, dtype == NSA_FP16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3,
                   const_cast<void*>(ptr), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  NSA_REQUIRE(r == CUDA_SUCCESS, NSA_ERR_CUDA, "cuTensorMapEncodeTiled failed with %d", (int)r);
  return NSA_OK;
}

bool attention_fwd_tc5_supports(const nsa_fwd_args& a) {
  const bool in8 = a.q_dtype == NSA_FP8_E4M3 || a.q_dtype == NSA_FP8_E5M2;
  if (!(a.q_dtype == NSA_BF16 || a.q_dtype == NSA_FP16 || in8)) return false;
  if (a.kv_dtype != a.q_dtype && !(in8 && a.kv_dtype == NSA_BF16)) return false;   // fp8 Q may come with bf16 K/V
  if (in8 && !(a.q_scale > 0.f && a.k_scale > 0.f && a.v_scale > 0.f)) return false;
  if (!(a.D == 64 || a.D == 128)) return false;
  if (!(a.scale > 0.f)) return false;
  if (a.branches & NSA_BRANCH_SELECTED) {
    if (a.bm != 64 || a.bn != 64 || a.top_k > T5_MAX_SEL) return false;
  }
  if ((a.branches & NSA_BRANCH_COMPRESSED) && a.Nc <= 0) return false;
  return true;
}

// The persistent variant runs the unsplit launches of ONE branch on 16-bit storage (the forward of the autograd route:
// measured 2-7 % faster there, T=65536, Hq=64, Hkv=4, D=128: compressed 4.53 against 4.61 ms, selected 2.63 against
// 2.72, sliding 1.93 against 2.02); launches of several branches are 1-4 % slower on it than on the one-item kernel
// (all three: 8.91-9.25 against 8.54-8.89 ms on the same box) and stay there, as do the split and fp8 launches.
// NSA_TC5_PERSIST=0 / =1 in the environment forces the one-item / the persistent kernel for every unsplit 16-bit launch.
// NSA_TC5_POLY=0 keeps every exponential on the special-function unit; default: 3 of 8 on the FMA pipe in unmasked tiles.
static int tc5_poly_mode() {
  static const int mode = [] { const char* e = getenv("NSA_TC5_POLY"); return !e ? 1 : (e[0] == '0' ? 0 : 1); }();
  return mode;
}
static int tc5_persistent_mode() {
  static const int mode = [] { const char* e = getenv("NSA_TC5_PERSIST"); return !e ? -1 : (e[0] == '0' ? 0 : 1); }();
  return mode;
}

int attention_fwd_tc5(const nsa_fwd_args& a, cudaStream_t st) {
  Tc5Params p;
  p.a = a;
  if (!(a.branches & NSA_BRANCH_SELECTED)) p.a.nq = (a.Tq + 63) / 64;
  const bool in8 = a.q_dtype == NSA_FP8_E4M3 || a.q_dtype == NSA_FP8_E5M2;
  const int cdt = in8 ? NSA_BF16 : a.q_dtype;             // type of the staged 16-bit tiles
  for (int br = 0; br < 3; ++br) {
    p.scale_log2[br] = a.scale * kLog2e;
    p.out_scale[br] = 1.f;
  }
  p.nk_blocks = (a.sel_key_limit + 63) / 64;
  {
    const int G = a.H / a.Hkv;
    p.GH = G % 4 == 0 ? 4 : (G % 2 == 0 ? 2 : 1);
    p.HG = G / p.GH;
  }
  int rc;
  p.kv8 = in8 && a.kv_dtype == a.q_dtype;
  p.poly = tc5_poly_mode();
  // NSA_TC5_KEEP_SUM=0: every branch end writes the whole running sum to the output row
  static const int psum_env = [] { const char* e = getenv("NSA_TC5_KEEP_SUM"); return !e ? 1 : (e[0] == '0' ? 0 : 1); }();
  p.psum = (psum_env && !in8 && !((a.nsplit > 1 || a.dyn_len != nullptr) && a.fused)) ? 1 : 0;
  p.fin_tma = 0;
  p.tma_out = 0;
  if (in8) rc = make_map8(&p.tmQ, a.Q, (long long)a.B * a.H, a.Tq, a.D);
  else rc = make_map(&p.tmQ, a.Q, (long long)a.B * a.H, a.Tq, a.D, cdt);
  if (rc != NSA_OK) return rc;
  if (p.kv8) {
    if ((rc = make_map8(&p.tmK, a.K, (long long)a.B * a.Hkv, a.Tk, a.D)) != NSA_OK) return rc;
    if ((rc = make_map8(&p.tmV, a.V, (long long)a.B * a.Hkv, a.Tk, a.D)) != NSA_OK) return rc;
  } else {
    if ((rc = make_map(&p.tmK, a.K, (long long)a.B * a.Hkv, a.Tk, a.D, cdt)) != NSA_OK) return rc;
    if ((rc = make_map(&p.tmV, a.V, (long long)a.B * a.Hkv, a.Tk, a.D, cdt)) != NSA_OK) return rc;
  }
  if (a.branches & NSA_BRANCH_COMPRESSED) {
    if ((rc = make_map(&p.tmKc, a.Kc, (long long)a.B * a.Hkv, a.Nc, a.D, cdt)) != NSA_OK) return rc;
    if ((rc = make_map(&p.tmVc, a.Vc, (long long)a.B * a.Hkv, a.Nc, a.D, cdt)) != NSA_OK) return rc;
  } else {
    p.tmKc = p.tmK;
    p.tmVc = p.tmV;
  }
  // NSA_TC5_FIN_TMA=0: the last branch end stores its rows thread by thread
  static const int fin_env = [] { const char* e = getenv("NSA_TC5_FIN_TMA"); return !e ? 1 : (e[0] == '0' ? 0 : 1); }();
  if (fin_env && p.psum && a.D == 128 && (reinterpret_cast<uintptr_t>(a.out) & 15) == 0) {
    auto enc = encode_fn();
    NSA_REQUIRE(enc != nullptr, NSA_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    // dims in ascending stride order: (D, Tq, H, B) for [B,H,Tq,D], (D, H, Tq, B) for [B,Tq,H,D]; the kernel swaps the two middle coordinates
    const bool bthd = (a.io_layout & NSA_IO_OUT_BTHD) != 0;
    const cuuint64_t D2 = (cuuint64_t)a.D * 2;
    cuuint64_t dims[4] = {(cuuint64_t)a.D, (cuuint64_t)(bthd ? a.H : a.Tq), (cuuint64_t)(bthd ? a.Tq : a.H), (cuuint64_t)a.B};
    cuuint64_t strides[3] = {D2, D2 * (cuuint64_t)(bthd ? a.H : a.Tq), D2 * a.Tq * a.H};
    cuuint32_t box[4] = {64, bthd ? 1u : 32u, bthd ? 32u : 1u, 1};
    cuuint32_t es[4] = {1, 1, 1, 1};
    CUresult r = enc(&p.tmOf, cdt == NSA_FP16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, a.out, dims,
                     strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    NSA_REQUIRE(r == CUDA_SUCCESS, NSA_ERR_CUDA, "cuTensorMapEncodeTiled (output, last write) failed with %d", (int)r);
    p.fin_tma = 1;
  }
  p.NQG = (p.a.nq + 4 / p.GH - 1) / (4 / p.GH);
  const long long items = (long long)p.NQG * a.B * a.Hkv * p.HG;
  // split launch: asked for by the caller (who supplies the scratch), fused bf16/fp16 forward only
  const bool split = (a.nsplit > 1 || a.dyn_len != nullptr) && a.fused && !in8;
  NSA_REQUIRE(a.dyn_len == nullptr || (split && a.causal), NSA_ERR_UNSUPPORTED,
              "attention forward: a device-resident length needs a fused, causal launch with 16-bit storage");
  p.nsplit = split ? (a.nsplit > 1 ? a.nsplit : 1) : 1;
  p.part = split ? reinterpret_cast<float*>(a.split_scratch) : nullptr;
  const long long rows = (long long)a.B * a.H * a.Tq;
  if (split) {
    const long long need = rows * p.nsplit * 3 * (a.D + 4) * 4;
    NSA_REQUIRE(a.split_scratch != nullptr && a.split_scratch_bytes >= need, NSA_ERR_ARG,
                "attention forward: a launch split %d ways needs %lld bytes of scratch, %lld given", p.nsplit, need,
                (long long)a.split_scratch_bytes);
    NSA_REQUIRE((reinterpret_cast<uintptr_t>(a.split_scratch) & 15) == 0, NSA_ERR_ARG, "attention forward: scratch must be 16-byte aligned");
  }
  const long long blocks = items * p.nsplit;
  NSA_REQUIRE(blocks > 0 && blocks < 2147483647LL, NSA_ERR_ARG, "attention forward: %lld work items do not fit a grid", blocks);
  const size_t smem = (size_t)(2 + 2 + 2) * (a.D / 64) * 128 * 128 + (in8 ? (size_t)2 * 128 * a.D : 0) + (p.psum ? 256 * 128 : 0) + 1024;
#define NSA_TC5_LAUNCH(DD, FF, I8, SP)                                                                     \
  {                                                                                                         \
    auto fn = nsa_fwd_tc5_kernel<DD, FF, I8, SP>;                                                           \
    NSA_CUDA_OK(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));         \
    fn<<<(unsigned)blocks, T5_THREADS, smem, st>>>(p);                                                     \
  }
  const int fmt = cdt == NSA_BF16 ? 1 : 0;
  if (split) {
    if (a.D == 128 && fmt == 1) NSA_TC5_LAUNCH(128, 1, false, true)
    else if (a.D == 128) NSA_TC5_LAUNCH(128, 0, false, true)
    else if (fmt == 1) NSA_TC5_LAUNCH(64, 1, false, true)
    else NSA_TC5_LAUNCH(64, 0, false, true)
    int rc2 = launch_status("attn_fwd_tc5 (split)");
    if (rc2 != NSA_OK) return rc2;
    const unsigned cgrid = (unsigned)((rows + 7) / 8);
#define NSA_TC5_COMBINE(TT, DD)                                                                                        \
    nsa_split_combine_kernel<TT, DD><<<cgrid, 256, 0, st>>>(p.part, reinterpret_cast<TT*>(a.out), a.gates, a.gate_dtype, \
                                                            a.gate_act, a.io_layout, a.H, a.Tq, rows, p.nsplit,       \
                                                            p.out_scale[0], p.out_scale[1], p.out_scale[2])
    if (a.D == 128 && fmt == 1) NSA_TC5_COMBINE(__nv_bfloat16, 128);
    else if (a.D == 128) NSA_TC5_COMBINE(__half, 128);
    else if (fmt == 1) NSA_TC5_COMBINE(__nv_bfloat16, 64);
    else NSA_TC5_COMBINE(__half, 64);
#undef NSA_TC5_COMBINE
    return launch_status("split_combine");
  }
  const int n_br = ((a.branches >> 0) & 1) + ((a.branches >> 1) & 1) + ((a.branches >> 2) & 1);
  if (!in8 && (tc5_persistent_mode() == 1 || (tc5_persistent_mode() == -1 && n_br == 1))) {
    // one thread block per SM walking the items (see nsa_fwd_tc5_persist_kernel)
    int dev = 0, sms = 0;
    NSA_CUDA_OK(cudaGetDevice(&dev));
    NSA_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    const unsigned grid = (unsigned)(blocks < sms ? blocks : sms);
    // results of single-branch items leave through the TMA (NSA_TC5_TMA_OUT=0 keeps the per-row stores)
    static const int tma_out_env = [] { const char* e = getenv("NSA_TC5_TMA_OUT"); return !e ? 1 : (e[0] == '0' ? 0 : 1); }();
    p.tma_out = 0;
    if (tma_out_env && (reinterpret_cast<uintptr_t>(a.out) & 15) == 0) {
      auto enc = encode_fn();
      NSA_REQUIRE(enc != nullptr, NSA_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
      // dims in ascending stride order: (D, Tq, H, B) for [B,H,Tq,D], (D, H, Tq, B) for [B,Tq,H,D]; the kernel swaps the two middle coordinates
      const bool bthd = (a.io_layout & NSA_IO_OUT_BTHD) != 0;
      const cuuint64_t D2 = (cuuint64_t)a.D * 2;
      cuuint64_t dims[4] = {(cuuint64_t)a.D, (cuuint64_t)(bthd ? a.H : a.Tq), (cuuint64_t)(bthd ? a.Tq : a.H), (cuuint64_t)a.B};
      cuuint64_t strides[3] = {D2, D2 * (cuuint64_t)(bthd ? a.H : a.Tq), D2 * a.Tq * a.H};
      cuuint32_t box[4] = {32, bthd ? 1u : 32u, bthd ? 32u : 1u, 1};
      cuuint32_t es[4] = {1, 1, 1, 1};
      CUresult r = enc(&p.tmO, cdt == NSA_FP16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, a.out, dims,
                       strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B,
                       CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
      NSA_REQUIRE(r == CUDA_SUCCESS, NSA_ERR_CUDA, "cuTensorMapEncodeTiled (output) failed with %d", (int)r);
      p.tma_out = 1;
    }
    const size_t smem_p = (size_t)(2 + 2 + 2) * (a.D / 64) * 128 * 128 + (p.tma_out ? 8 * 2048 : 0) + 1024;
#define NSA_TC5_PERSIST_LAUNCH(DD, FF)                                                                     \
  {                                                                                                         \
    auto fn = nsa_fwd_tc5_persist_kernel<DD, FF>;                                                           \
    NSA_CUDA_OK(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_p));       \
    fn<<<grid, T5_THREADS, smem_p, st>>>(p, (int)blocks);                                                  \
  }
    if (a.D == 128 && fmt == 1) NSA_TC5_PERSIST_LAUNCH(128, 1)
    else if (a.D == 128) NSA_TC5_PERSIST_LAUNCH(128, 0)
    else if (fmt == 1) NSA_TC5_PERSIST_LAUNCH(64, 1)
    else NSA_TC5_PERSIST_LAUNCH(64, 0)
#undef NSA_TC5_PERSIST_LAUNCH
    return launch_status("attn_fwd_tc5 (persistent)");
  }
  if (in8 && a.D == 128) NSA_TC5_LAUNCH(128, 1, true, false)
  else if (in8) NSA_TC5_LAUNCH(64, 1, true, false)
  else if (a.D == 128 && fmt == 1) NSA_TC5_LAUNCH(128, 1, false, false)
  else if (a.D == 128) NSA_TC5_LAUNCH(128, 0, false, false)
  else if (fmt == 1) NSA_TC5_LAUNCH(64, 1, false, false)
  else NSA_TC5_LAUNCH(64, 0, false, false)
#undef NSA_TC5_LAUNCH
  return launch_status("attn_fwd_tc5");
}

// Synchronises `st`, returns and clears the status word the tcgen05 kernels set when a bounded wait gave up.
int tc5_take_status(cudaStream_t st, int* status) {
  NSA_CUDA_OK(cudaStreamSynchronize(st));
  int v = 0, zero = 0;
  NSA_CUDA_OK(cudaMemcpyFromSymbol(&v, g_tc5_status, sizeof(int)));
  if (v != 0) NSA_CUDA_OK(cudaMemcpyToSymbol(g_tc5_status, &zero, sizeof(int)));
  *status = v;
  return NSA_OK;
}

int tc5_set_status(int v) {
  NSA_CUDA_OK(cudaMemcpyToSymbol(g_tc5_status, &v, sizeof(int)));
  return NSA_OK;
}

}  // namespace nsa
