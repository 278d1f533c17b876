// Tensor-core forward of alpha-entmax attention and Lazy Attention: one CTA per 128-row
// query tile, warp-specialised.
//
//   warps 0-15  row threads.  Key tiles alternate between two groups (group g = tiles whose running
//               index is congruent to g mod 2, score buffers g and g + 2); inside a group two
//               threads share a query row, 64 of a tile's 128 keys each.  They read the score tile
//               from tensor memory and accumulate the row statistics (entmax: max, then
//               Halley/Newton iterations on tau; lazy: online log-sum-exp); the four partial results
//               of a row meet in shared memory at the end of a pass.  In the last pass P (bf16/fp16)
//               goes to a tensor-memory buffer of its own and becomes the A operand of P.V;
//   warp 16     TMA producer: Q once, then K (and in the last pass V) tiles through a ring;
//   warps 17,18 tcgen05.mma issuers: in the score passes one tile each in turn, in the last pass one
//               issues S = Q.K^T, the other O += P.V.
//
// Tensor-memory columns.  Score passes: four score buffers [128 b, 128 b + 128).  Last pass: S(t) in
// buffer t & 1, O at [256, 256 + D), probabilities of tile t at [384 + 64 (t & 1), +64).
//
// Replaces lazy_attention_triton.py:9-174 (LSE + output kernels) for Lazy Attention and the
// adasplash forward (source absent from the reference checkout) for entmax attention.
#pragma once

#include "common.cuh"
#include "tc_prims.cuh"

namespace fla {
namespace tc {

constexpr int kGroupThreads = 128;     // one row per thread
constexpr int kComputeThreads = 256;   // two groups
constexpr int kProducerWarp = 8;
constexpr int kMmaWarp = 9;
// forward kernel: 16 row warps (two tile groups x two column halves), the copy producer, two issuers
constexpr int kFwdRowThreads = 512;
constexpr int kFwdBufWarps = 8;        // warps reading one score buffer: one arrival each
constexpr int kFwdProducerWarp = 16;
constexpr int kFwdMmaWarp = 17;
constexpr int kFwdThreads = 608;
constexpr uint32_t kProbCol = 384;     // last pass: probability buffers at tensor-memory columns 384 + 64 g
constexpr int kMaxMaskWords = 64;  // block-mask words per query block: L <= 131072
// Candidates of the entmax forward: every row thread keeps the scores that can still lie above the row's
// threshold in kStageSlots private shared-memory slots.
constexpr int kStageSlots = 24;
constexpr int kStageKeep = 16;    // most a thread keeps after tightening: 8 slots stay free for the next 8 scores
constexpr int kPoolSize = 256;    // spill pool of a CTA, (value, row) pairs
constexpr int kStageBytes = kStageSlots * kFwdRowThreads * 4;

template <int D>
struct TileCfg {
  static constexpr int kBoxBytes = 128 * 128;            // 128 rows x 64 elements x 2 bytes
  static constexpr int kBoxes = D / 64;
  static constexpr int kTileBytes = kBoxes * kBoxBytes;  // a 128 x D tile
  // Ring depth.  Even on purpose: the two issuing threads take alternate tiles, so with an even
  // depth every ring slot is always consumed by the same thread.  A parity wait is only sound for
  // a waiter that sees every phase of its barrier; with an odd depth a thread would wait for fill
  // n+1 of a slot whose fill n went to the other thread, and pass while fill n is still in flight.
  static constexpr int kStages = D == 128 ? 4 : 8;
  static_assert(kStages % 2 == 0 && (kStages & (kStages - 1)) == 0, "ring depth must be an even power of two");
  static constexpr int kKSteps = D / 16;
};

struct FwdShared {
  uint64_t q_full, ring_full[8], ring_empty[8], s_full[4], s_free[4], f_full[2], p_full[2], pv_done[2], pass_done, o_full;
  uint32_t tmem_base;
  int abort_flag;
  int cont_flag;
  uint32_t mask_words[kMaxMaskWords];
  float part[4][3][128];   // per (group, half), per statistic, per row: partial row sums of a pass
  // Key tiles still worth visiting.  tau rises monotonically from the left end of its bracket, so
  // a tile without any score above the current tau stays without one: the row threads mark the
  // tiles with a positive entry during a pass (act_next), the next pass and the last pass visit
  // only those (act[parity of the pass]; two copies, so that the producer and the issuer may still
  // scan the bitmap of a pass while the row threads publish the next one).  After a step in which
  // some row's tau fell, the next pass visits the tiles marked during the first threshold pass
  // (act_base: entries above max - 1, the lower end of every row's bracket) instead.
  uint32_t act[2][32], act_next[32], act_base[32];
  uint64_t pass_ack;   // the producer and both issuers have read the verdict of the last pass
  int force_all;
  // Running score maximum of each of the four threads of a row during the row-max pass.  Read by
  // the other three without synchronisation: a stale value is a smaller one, and any lower bound of
  // the row maximum keeps the candidate filter below a superset filter.
  float rmax[4][128];
  // The same for the lower bound of the row's threshold each of the four threads derived from its own
  // candidates ((alpha-1)*score units): any of them, stale or not, is a valid lower bound.
  float rlb[4][128];
  // ... and a tangent (value at 0, slope) of each thread's part of f, see the row-max pass.
  float2 rtan[4][128];
  // Spill pool: (score, row) pairs of threads that were left with more than kStageKeep candidates.
  float2 pool[kPoolSize];
  int npool;
};

template <int D>
__device__ __forceinline__ void tma_load_tile(uint8_t* dst, const CUtensorMap* map, uint64_t* bar, int row, int h,
                                              int b) {
#pragma unroll
  for (int box = 0; box < TileCfg<D>::kBoxes; ++box)
    tma_load_4d(dst + box * TileCfg<D>::kBoxBytes, map, bar, box * 64, row, h, b);
}

// S[128 x 128] = A[128 x D] . B[128 x D]^T, both operands K-major tiles in shared memory.
template <int D, int FMT>
__device__ __forceinline__ void issue_nt(uint32_t d_tmem, uint32_t a_addr, uint32_t b_addr) {
  constexpr uint32_t idesc = make_idesc(128, 128, FMT, 0, 0);
#pragma unroll
  for (int ks = 0; ks < TileCfg<D>::kKSteps; ++ks) {
    const uint32_t off = (ks >> 2) * TileCfg<D>::kBoxBytes + (ks & 3) * 32;
    umma_ss(d_tmem, desc_kmajor(a_addr + off), desc_kmajor(b_addr + off), idesc, ks > 0);
  }
}

// kind::f16 products need A and B in the same 16-bit format: an fp16 A operand next to a bf16 B
// operand raises an illegal-instruction error on sm_100a, so probabilities are rounded to the
// input type.

// O[128 x D] (+)= A[128 x 128] . B[128 x D]: A in tensor memory (two 16-bit values per column,
// format AFMT), B a [128 rows x D] tile in shared memory (format FMT) whose rows are the
// reduction dimension (MN-major).
// `nks` (1..8): number of 16-row steps of the reduction dimension to issue; fewer than 8 for the one
// tile that reaches beyond the end of a sequence (see zero_tail_rows).
template <int D, int AFMT, int FMT>
__device__ __forceinline__ void issue_tn(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_addr, bool accumulate,
                                         int nks = 8) {
  constexpr uint32_t idesc = make_idesc2(128, D, AFMT, FMT, 0, 1);
#pragma unroll
  for (int ks = 0; ks < 8; ++ks)
    if (ks < nks)
      umma_ts(d_tmem, a_tmem + ks * 8, desc_mnmajor(b_addr + ks * 2048, TileCfg<D>::kBoxBytes), idesc,
              (accumulate || ks > 0) ? 1u : 0u);
}

// D[128 x D] (+)= A[128 x 128] . B[128 x D]: A in tensor memory as four pieces of 16 columns (16-bit
// pairs), piece q at a_tmem + 32 q (each of the four threads of a row writes its 32 reduction elements inside
// the columns it read); B a [128 rows x D] tile whose rows are the reduction dimension.  `nks`: 16-row steps
// to issue (fewer than 8 for the tile that reaches into a sequence's padding).
template <int D, int FMT>
__device__ __forceinline__ void issue_tn_quads(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_addr, bool accumulate,
                                               int nks = 8) {
  constexpr uint32_t idesc = make_idesc(128, D, FMT, 0, 1);
#pragma unroll
  for (int ks = 0; ks < 8; ++ks)
    if (ks < nks)
      umma_ts(d_tmem, a_tmem + 32 * (ks >> 1) + 8 * (ks & 1), desc_mnmajor(b_addr + ks * 2048, TileCfg<D>::kBoxBytes), idesc,
              (accumulate || ks > 0) ? 1u : 0u);
}

// Rows of q, k, v, dO at or beyond a sequence's length are padding and may hold anything, NaN
// included (the reference masks every load, lazy_attention_triton.py:41,56,171,215-232).  A score
// computed from a padding row is replaced by the row threads before it is used, but a tile that is
// the reduction operand of a second product (V in P.V, K in dS.K, Q and dO in dS^T.Q and P^T.dO)
// would multiply its padding by the zeros standing in the other operand, and 0 * NaN is NaN.  So
// for the one tile of a sequence that straddles its end, the issuing thread leaves the reduction
// steps that lie wholly in the padding away (`nks` above) and clears the padding rows of the last,
// partial step in shared memory before it issues.  Row r of a tile occupies bytes [128 r, 128 r + 128)
// of every 64-column box, whatever the swizzle.  `rows_per_box`: 128, or 64 for the sub-tiles of the
// dK/dV kernel.  Returns the number of 16-row steps to issue.
__device__ __forceinline__ int zero_tail_rows(uint8_t* tile, int valid_rows, int boxes, int rows_per_box) {
  const int nks = (valid_rows + 15) >> 4;
  const int r1 = min(nks * 16, rows_per_box);
  if (valid_rows < r1) {
    for (int box = 0; box < boxes; ++box) {
      uint4* row = (uint4*)(tile + (size_t)box * rows_per_box * 128 + (size_t)valid_rows * 128);
      for (int x = 0; x < (r1 - valid_rows) * 8; ++x) row[x] = make_uint4(0u, 0u, 0u, 0u);
    }
    fence_proxy_async_smem();   // generic-proxy stores before the tensor core's reads
  }
  return nks;
}

__device__ __forceinline__ uint8_t* align_1024(uint8_t* p) {
  return (uint8_t*)(((uintptr_t)p + 1023) & ~(uintptr_t)1023);
}

// Convergence threshold on the change of tau between two iterations (tau - max is in [-1, 0)).
// A row stops iterating once a regular (not bisected) step is this short.  The step that follows
// a Halley step of length d is of order d^3 (alpha <= 1.5), the one after a Newton step of order
// d^2: with these limits the threshold that is kept lies within a few 1e-5 of the root (measured on
// Gaussian and heavy-tailed rows up to 8192 keys), far below the resolution of 16-bit
// probabilities, and one whole pass over the keys is saved against a limit of 1e-4.
constexpr float kTauTolHalley = 1e-2f;
constexpr float kTauTolNewton = 1e-3f;
constexpr float kTauTol = 1e-4f;   // after a bisected step
// The same limits for the iteration on candidate lists, where one more iteration is cheap.
constexpr float kListTolHalley = 1e-3f;
constexpr float kListTolNewton = 1e-4f;
constexpr float kListTol = 1e-5f;



// 8-byte shared-memory accesses that are not cached in registers: other warps write these pairs.
__device__ __forceinline__ float2 lds_f2(const float2* ptr) {
  float2 v;
  asm volatile("ld.volatile.shared.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(smem_u32(ptr)) : "memory");
  return v;
}
__device__ __forceinline__ void sts_f2(float2* ptr, float a, float b) {
  asm volatile("st.volatile.shared.v2.f32 [%0], {%1, %2};" ::"r"(smem_u32(ptr)), "f"(a), "f"(b) : "memory");
}

// Streaming candidates of the entmax forward (see the row-max pass of fwd_kernel): Newton steps from the
// left on "my candidates exactly + the tangents the other three threads of the row published - 1", then
// publish my tangent and bound, and drop the candidates the bound excludes.  A thread left with more than
// kStageKeep candidates hands the surplus to the CTA's spill pool (a rare event: the tail of how a row's
// support splits over its four threads); `kept` = -1 reports that the pool is full.  Not inlined: it is
// called from two places inside the hottest loop of the kernel and would otherwise take its registers.
struct TightenResult { float bound; int kept; };
template <int KIND>
static __device__ __noinline__ TightenResult tighten_candidates(FwdShared* sh, float* stage_t, int n_st, float t, float c1,
                                                               float e, int quad, int row, int steps, int keep_if) {
  // (few registers on purpose: a call that has to save many of its caller's registers goes through local
  // memory, and with almost all of the SM's memory configured as shared memory that means L2)
  // the other threads' tangents: sum_j [X_j - t]_+^e >= oc + ob * t over their candidates
  float oc = 0.f, ob = 0.f;
#pragma unroll
  for (int qq = 0; qq < 4; ++qq) {
    const float2 tg = lds_f2(&sh->rtan[qq][row]);   // (one 8-byte load: a pair is never torn)
    if (qq != quad) { oc += tg.x; ob += tg.y; }
  }
  float te = t, s0 = 0.f, s1 = 0.f;
#pragma unroll 1
  for (int it = 0; it < steps; ++it) {
    te = t; s0 = 0.f; s1 = 0.f;
#pragma unroll 2
    for (int j = 0; j < n_st; ++j) {
      const float d = fmaf(stage_t[j * kFwdRowThreads], c1, -t);   // <= 1: t >= (row maximum so far) - 1
      if (KIND == 0) { const float ee = __saturatef(d); s0 = fmaf(ee, ee, s0); s1 += ee; }
      else if (KIND == 1) { s0 += fmaxf(d, 0.f); s1 += d > 0.f ? 1.f : 0.f; }
      else if (d > 0.f) { float pw, u; p_and_u<2>(d, e, pw, u); s0 += pw; s1 += u; }
    }
    const float fv = s0 + fmaf(ob, t, oc) - 1.f;              // <= f(t) of the whole row
    const float tn = t + __fdividef(fv, fmaf(e, s1, -ob));     // slope -(e s1 - ob) < 0
    if (!(fv > 0.f) || !(tn > t)) break;
    t = tn;
  }
  // my tangent at the last point evaluated: s0 - e s1 (t - te)
  sts_f2(&sh->rtan[quad][row], fmaf(e * s1, te, s0), -e * s1);
  ((volatile float*)&sh->rlb[0][0])[quad * 128 + row] = t;
  int k = n_st;
  if (n_st > keep_if) {
    k = 0;
#pragma unroll 1
    for (int j = 0; j < n_st; ++j) {
      const float v = stage_t[j * kFwdRowThreads];
      if (fmaf(v, c1, -t) > 0.f) { stage_t[k * kFwdRowThreads] = v; ++k; }
    }
    if (k > kStageKeep) {   // hand the surplus to the pool
      for (int j = kStageKeep; j < k; ++j) {
        const int pos = atomicAdd(&sh->npool, 1);
        if (pos < kPoolSize) sh->pool[pos] = make_float2(stage_t[j * kFwdRowThreads], __int_as_float(row));
        else k = -1 - kStageSlots;   // pool full
      }
      k = k < 0 ? -1 : kStageKeep;
    }
  }
  TightenResult r;
  r.bound = t;
  r.kept = k;
  return r;
}

// LISTS: the entmax row-max pass keeps candidates and the thresholds are iterated on them (otherwise: by
// passes over recomputed score tiles only).  A compile-time switch, because the candidate bookkeeping costs
// the pass-only kernel registers it does not have.
// PAIR (entmax, thresholds by score passes only): one CTA holds TWO adjacent query tiles.  A K tile fetched from L2
// then serves two score products -- the score passes are bound by that fetch -- and row group g works on the rows
// of query tile g for every key tile (without PAIR the groups split the key tiles of one query tile between them).
// With the running tile index t of a pass mapped to 2 t + g for group and issuer g, the buffer and barrier
// arithmetic of the score passes is the same in both forms.  The last pass runs once per query tile, one after the
// other (tensor memory holds one output accumulator).
template <int MODE, int D, int FMT, int KIND, bool LISTS, bool PAIR = false>
__global__ void __launch_bounds__(kFwdThreads, 1)
fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
           const __grid_constant__ CUtensorMap map_v, const AttnParams p, int* status) {
  using Cfg = TileCfg<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align_1024(smem_raw);
  static_assert(!PAIR || (MODE == ENTMAX && !LISTS), "the two-tile form exists for entmax score passes only");
  constexpr int NQ = PAIR ? 2 : 1;   // query tiles of this CTA
  uint8_t* sQ = smem;
  uint8_t* ring = smem + NQ * Cfg::kTileBytes;
  uint8_t* stage = ring + Cfg::kStages * Cfg::kTileBytes;   // entmax only: candidate slots of the row threads
  __shared__ FwdShared sh;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool causal = (MODE == LAZY) ? true : (p.causal != 0);
  const int L = p.L;
  const int nmt = (L + 127) >> 7;
  const int BH = p.B * p.H;
  // heaviest query tiles (largest index under the causal mask) are scheduled first
  // All query tiles of one (batch, head) pair are adjacent in the grid, heaviest first: the CTAs in
  // flight at any time stream the same few K/V tensors, which therefore stay in the L2 cache.
  // (With the pair as the fast index every resident CTA would stream a different pair from HBM.)
  const int ncta = PAIR ? (nmt + 1) >> 1 : nmt;    // CTAs per (batch, head) pair
  const int bh = (int)(blockIdx.x / ncta);
  const int mt = NQ * (ncta - 1 - (int)(blockIdx.x % ncta));   // (first) query tile of this CTA
  const int b = bh / p.H, h = bh % p.H;
  const int len = p.varlen ? min(max(p.varlen[b], 0), L) : L;
  const int row0 = mt * 128;
  const bool tile_live = row0 < len;
  // key tiles the CTA visits: those the last of its live query tiles may look at
  const int mt_hi = (PAIR && row0 + 128 < len) ? mt + 1 : mt;
  const int nkt = tile_live ? (causal ? min((len + 127) >> 7, mt_hi + 1) : ((len + 127) >> 7)) : 0;
  const int nsub = tile_live ? (mt_hi - mt + 1) : 0;   // live query tiles of this CTA
  volatile int* abort_flag = &sh.abort_flag;
  if (tid == 0) kernel_clock(status, 0, false);

  if (tid == 0) {
    mbar_init(&sh.q_full, 1);
    // (two-tile form: a K tile is released by the commits of both issuers; in its last passes the one issuer
    // that reads a slot commits twice)
    for (int s = 0; s < 8; ++s) { mbar_init(&sh.ring_full[s], 1); mbar_init(&sh.ring_empty[s], PAIR ? 2 : 1); }
    for (int s = 0; s < 4; ++s) {
      mbar_init(&sh.s_full[s], 1);
      mbar_init(&sh.s_free[s], kFwdBufWarps);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&sh.f_full[s], 1);
      mbar_init(&sh.p_full[s], kFwdBufWarps);
      mbar_init(&sh.pv_done[s], 1);
    }
    mbar_init(&sh.pass_done, 1);
    mbar_init(&sh.pass_ack, 3);
    mbar_init(&sh.o_full, PAIR ? 2 : 1);   // (two-tile form: one commit per issuer)
    sh.abort_flag = 0;
    sh.cont_flag = 0;
    fence_mbar_init();
  }
  if (tid < kMaxMaskWords) {
    sh.mask_words[tid] = 0;
    if (PAIR) reinterpret_cast<uint32_t*>(stage)[tid] = 0;   // (block-mask words of the second query tile)
  }
  if (tid < kFwdRowThreads) {
    (&sh.rmax[0][0])[tid] = -INFINITY;
    (&sh.rlb[0][0])[tid] = -INFINITY;
    (&sh.rtan[0][0])[tid] = make_float2(0.f, 0.f);
  }
  if (tid < 32) {
    const int lo = tid * 32;
    sh.act[0][tid] = sh.act[1][tid] = nkt >= lo + 32 ? 0xffffffffu : (nkt > lo ? (1u << (nkt - lo)) - 1u : 0u);
    sh.act_next[tid] = 0u;
    if (tid == 0) { sh.force_all = 0; sh.npool = 0; }
  }
  if (warp == kFwdProducerWarp) tmem_alloc(&sh.tmem_base, 512);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = sh.tmem_base;
  const uint32_t tmem_o = tmem + 256;
  // Visits the key tiles a pass works on: fn(kt).  Ascending order, except for the row-max pass of
  // entmax (pass 0), which starts at the last tile: under a causal mask that is the diagonal, where
  // the largest scores of a row tend to sit, and the sooner the running maximum is close to the final
  // one the fewer tiles that pass marks for the threshold passes.
  auto for_each_tile = [&](uint32_t pass, auto&& fn) {
    const volatile uint32_t* words = (const volatile uint32_t*)sh.act[pass & 1u];
    const int nwords = (nkt + 31) >> 5;
    if (MODE == ENTMAX && pass == 0) {
      for (int w = nwords - 1; w >= 0; --w) {
        uint32_t bits = words[w];
        while (bits) {
          const int bit = 31 - __clz((int)bits);
          bits &= ~(1u << bit);
          fn(w * 32 + bit);
        }
      }
      return;
    }
    for (int w = 0; w < nwords; ++w) {
      uint32_t bits = words[w];
      while (bits) {
        const int bit = __ffs((int)bits) - 1;
        bits &= bits - 1u;
        fn(w * 32 + bit);
      }
    }
  };
  // Position in the ring of key/value tiles: a running count of the tiles that went through it.
  struct RingPos {
    uint32_t pos = 0;
    __device__ __forceinline__ uint32_t stage_at(uint32_t ofs) const { return (pos + ofs) & (uint32_t)(Cfg::kStages - 1); }
    __device__ __forceinline__ uint32_t phase_at(uint32_t ofs) const { return ((pos + ofs) / (uint32_t)Cfg::kStages) & 1u; }
    __device__ __forceinline__ uint32_t stage() const { return stage_at(0); }
    __device__ __forceinline__ uint32_t phase() const { return phase_at(0); }
    __device__ __forceinline__ void advance() { ++pos; }
  };
  // Order of the loads of the last pass: K(0), then K(t+1) before V(t).  The K tile of the next
  // score product never queues behind a V slot that is still waiting for its P.V product.
  // Offsets from the ring position at the start of the pass (n = number of tiles):
  auto fin_k_ofs = [](int t) { return (uint32_t)(t == 0 ? 0 : 2 * t - 1); };
  auto fin_v_ofs = [](int t, int n) { return (uint32_t)(t == n - 1 ? 2 * n - 1 : 2 * t + 2); };

  if (warp == kFwdProducerWarp) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0 && tile_live) {
      tma_prefetch_desc(&map_q);
      tma_prefetch_desc(&map_k);
      tma_prefetch_desc(&map_v);
      mbar_expect_tx(&sh.q_full, NQ * Cfg::kTileBytes);
      tma_load_tile<D>(sQ, &map_q, &sh.q_full, row0, h, b);
      if (PAIR) tma_load_tile<D>(sQ + Cfg::kTileBytes, &map_q, &sh.q_full, row0 + 128, h, b);   // (rows beyond L read as zeros)
      RingPos rp;
      uint32_t pass = 0;
      auto load = [&](const CUtensorMap* map, int kt, int tag) {
        // after an expired wait nothing more is issued: copies without flow control would overrun
        // the transaction counts of the barriers and land in shared memory that is being released
        const uint32_t st = rp.stage();
        if (!mbar_wait(&sh.ring_empty[st], rp.phase() ^ 1u, abort_flag, status, tag)) return;
        mbar_expect_tx(&sh.ring_full[st], Cfg::kTileBytes);
        tma_load_tile<D>(ring + st * Cfg::kTileBytes, map, &sh.ring_full[st], kt * 128, h / p.n_rep, b);   // (kv head)
        rp.advance();
      };
      while (true) {  // score-only passes
        for_each_tile(pass, [&](int kt) { load(&map_k, kt, 10); });
        mbar_wait(&sh.pass_done, pass & 1, abort_flag, status, 11);
        ++pass;
        const int go_on = *(volatile int*)&sh.cont_flag;
        mbar_arrive(&sh.pass_ack);
        if (!go_on || *abort_flag) break;
      }
      {   // last pass: K(0), K(1), V(0), K(2), V(1), ..., V(n-1)
        int prev = -1;
        for_each_tile(pass, [&](int kt) {
          load(&map_k, kt, 12);
          if (prev >= 0) load(&map_v, prev, 12);
          prev = kt;
        });
        if (prev >= 0) load(&map_v, prev, 12);
      }
    }
    __syncwarp();
  } else if (warp == kFwdMmaWarp || warp == kFwdMmaWarp + 1) {
    // ------------------------------------------------------------------ MMA issuers
    // Two threads (one per warp) issue the products.  A thread spends several hundred cycles per
    // tile on its waits, commits and loop, in sequence with the issue itself, which blocks while
    // the tensor pipe is busy; one thread alone leaves the pipe idle for that long after every
    // tile.  In the score passes the two take alternate tiles (issuer w feeds the score buffers of
    // row group w); in the last pass one issues the score products, the other the P.V products.
    if (lane == 0 && tile_live) {
      const uint32_t me = (uint32_t)(warp - kFwdMmaWarp);
      const uint32_t q_addr = smem_u32(sQ), ring_addr = smem_u32(ring);
      unsigned long long issued = 0;
      mbar_wait(&sh.q_full, 0, abort_flag, status, 20);
      RingPos rp;
      uint32_t sn = 0, pass = 0;
      while (true) {
        for_each_tile(pass, [&](int kt) {
          if (PAIR || (sn & 1u) == me) {
            const uint32_t vs = PAIR ? 2u * sn + me : sn;   // (two-tile form: every tile, for query tile `me`)
            const uint32_t sb = vs & 3u;   // four score buffers in flight
            const uint32_t st = rp.stage();
            bool ok = mbar_wait(&sh.ring_full[st], rp.phase(), abort_flag, status, 21);
            ok = ok && mbar_wait(&sh.s_free[sb], ((vs >> 2) & 1u) ^ 1u, abort_flag, status, 22);
            tc_fence_after_sync();
            if (ok) issue_nt<D, FMT>(tmem + sb * 128, q_addr + (PAIR ? me * Cfg::kTileBytes : 0u), ring_addr + st * Cfg::kTileBytes);
            umma_commit(&sh.ring_empty[st]);
            umma_commit(&sh.s_full[sb]);
            ++issued;
          }
          rp.advance();
          ++sn;
        });
        mbar_wait(&sh.pass_done, pass & 1, abort_flag, status, 23);
        ++pass;
        const int go_on = *(volatile int*)&sh.cont_flag;
        mbar_arrive(&sh.pass_ack);
        if (!go_on || *abort_flag) break;
      }
      // Last pass (every score buffer is free here: the row threads signalled the end of the last
      // score pass).  Tile t takes two ring slots, one for K and one for V (order of the loads:
      // see fin_k_ofs / fin_v_ofs); S(t) goes to score buffer t & 1 once the row threads have read
      // S(t-2) from there.  One thread issues the score products, the other one the P.V products;
      // whenever either starts to wait for a fill of a slot, the slot's previous fill has landed
      // (it was consumed by the same thread, or by a product that the waiter's last product
      // depended on).
      int nfin = 0;
      for (int w = 0; w * 32 < nkt; ++w) nfin += __popc(((volatile uint32_t*)sh.act[pass & 1u])[w]);
      const bool score_role = PAIR ? me == 0u : (sn & 1u) == me;
      // the last key tile of the sequence may reach into its padding: if it is visited at all, it is
      // visited last (ascending order)
      const int tail_valid = len - (nkt - 1) * 128;
      const bool tail_visited = nkt > 0 && tail_valid < 128 &&
                                ((((volatile uint32_t*)sh.act[pass & 1u])[(nkt - 1) >> 5] >> ((nkt - 1) & 31)) & 1u) != 0u;
      if constexpr (PAIR) {
        // Two-tile form: both query tiles go through the last pass together, on the same K and V tiles.  Issuer g
        // serves query tile g: S_g(t) into score buffer g, then -- once row group g has written P_g(t) over it --
        // O_g += P_g(t) . V(t), accumulators at columns 256 and 384.  A K or V slot is released by the commits of
        // both issuers.  The chain S -> P -> P.V -> next S of one query tile runs while the other tile's does.
        const uint32_t q_mine = q_addr + me * Cfg::kTileBytes, s_mine = tmem + me * 128, o_mine = tmem + 256 + me * 128;
        for (int t = 0; t < nfin; ++t) {
          const uint32_t ok_ofs = fin_k_ofs(t), ov_ofs = fin_v_ofs(t, nfin);
          const uint32_t stk = rp.stage_at(ok_ofs), stv = rp.stage_at(ov_ofs);
          bool ok = mbar_wait(&sh.ring_full[stk], rp.phase_at(ok_ofs), abort_flag, status, 24 + me);
          // P_g(t-1) stands in this buffer until its product has read it
          if (t >= 1) ok = ok && mbar_wait(&sh.pv_done[me], (uint32_t)(t - 1) & 1u, abort_flag, status, 28);
          tc_fence_after_sync();
          if (ok) issue_nt<D, FMT>(s_mine, q_mine, ring_addr + stk * Cfg::kTileBytes);
          umma_commit(&sh.ring_empty[stk]);
          umma_commit(&sh.f_full[me]);
          ok = ok && mbar_wait(&sh.p_full[me], (uint32_t)t & 1u, abort_flag, status, 26);
          ok = ok && mbar_wait(&sh.ring_full[stv], rp.phase_at(ov_ofs), abort_flag, status, 24 + me);
          tc_fence_after_sync();
          int nks = 8;
          // (both issuers clear the same padding rows with the same zeros)
          if (ok && tail_visited && t == nfin - 1) nks = zero_tail_rows(ring + stv * Cfg::kTileBytes, tail_valid, Cfg::kBoxes, 128);
          if (ok) issue_tn_quads<D, FMT>(o_mine, s_mine, ring_addr + stv * Cfg::kTileBytes, t > 0, nks);
          umma_commit(&sh.ring_empty[stv]);
          umma_commit(&sh.pv_done[me]);
          issued += 2;
        }
        umma_commit(&sh.o_full);
      } else {
        for (int t = 0; t < nfin; ++t) {
          const uint32_t sb = (uint32_t)t & 1u;
          const uint32_t ofs = score_role ? fin_k_ofs(t) : fin_v_ofs(t, nfin);
          const uint32_t st = rp.stage_at(ofs);
          bool ok = mbar_wait(&sh.ring_full[st], rp.phase_at(ofs), abort_flag, status, 24 + me);
          if (score_role) {
            // the row threads have read S(t-2) out of this buffer (their probabilities live elsewhere)
            if (t >= 2) ok = ok && mbar_wait(&sh.p_full[sb], ((t - 2) >> 1) & 1, abort_flag, status, 28);
            tc_fence_after_sync();
            if (ok) issue_nt<D, FMT>(tmem + sb * 128, q_addr, ring_addr + st * Cfg::kTileBytes);
            umma_commit(&sh.ring_empty[st]);
            umma_commit(&sh.f_full[sb]);
          } else {
            ok = ok && mbar_wait(&sh.p_full[sb], (t >> 1) & 1, abort_flag, status, 26);
            tc_fence_after_sync();
            int nks = 8;
            if (ok && tail_visited && t == nfin - 1) nks = zero_tail_rows(ring + st * Cfg::kTileBytes, tail_valid, Cfg::kBoxes, 128);
            if (ok) issue_tn<D, FMT, FMT>(tmem_o, tmem + kProbCol + sb * 64, ring_addr + st * Cfg::kTileBytes, t > 0, nks);
            umma_commit(&sh.ring_empty[st]);
            umma_commit(&sh.pv_done[sb]);
          }
          ++issued;
        }
        if (!score_role) umma_commit(&sh.o_full);
      }
      if (status) atomicAdd((unsigned long long*)(status + 4), issued);
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ row threads
    // Sixteen warps.  Tiles alternate between two groups (group g owns the score buffers g and
    // g + 2, i.e. every tile whose running index is congruent to g mod 2); inside a group two
    // threads share a row of the query tile, each taking 64 of the 128 keys of a tile (half 0 the
    // first 64).  Four warps per scheduler keep its arithmetic pipe busy while others wait for
    // a barrier or a tensor-memory load.  The partial row statistics of the four threads of a row
    // meet in shared memory at the end of a pass.
    const int grp = (warp >> 2) & 1;
    const int half = warp >> 3;
    const int quad = grp * 2 + half;
    const int c0 = half * 64;                  // first key column of this thread inside a tile
    const int row = (warp & 3) * 32 + lane;
    const int row0g = row0 + (PAIR ? grp * 128 : 0);   // first row of the query tile this thread's score passes work on
    const int i = row0g + row;
    const bool live = i < len;
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t tgrp = tmem + lane_base;   // + 128 * buffer index
    const int64_t bhl = (int64_t)bh * L;
    if (tile_live) {
      // key j is valid for this row iff j <= jlim
      const int jlim = live ? (causal ? min(i, len - 1) : len - 1) : -1;
      // tiles whose last key exceeds this bound hold masked entries for some row
      const int tile_jlim = (row0g + 127 < len) ? (causal ? row0g : len - 1) : -1;
      uint32_t sn = 0;    // running tile index at the start of the current pass
      uint32_t rpass = 0; // index of the current pass
      float rstat = 0.f;  // tau (entmax) or base-2 log-sum-exp (lazy)

      // A reader without a tile in some pass (one active tile: the other issuer takes it) must not
      // be lapped: the verdict of pass n is written only after all three readers took that of n-1.
      uint32_t signalled = 0;
      auto signal_pass = [&](bool cont) {
        if (tid == 0) {
          if (signalled > 0) mbar_wait(&sh.pass_ack, (signalled - 1u) & 1u, abort_flag, status, 35);
          ++signalled;
          *(volatile int*)&sh.cont_flag = cont ? 1 : 0;
          __threadfence_block();
          mbar_arrive(&sh.pass_done);
        }
      };
      // Visits the tiles of pass `pass` that belong to this thread's group: fn(kt, running index).
      auto for_my_tiles = [&](uint32_t pass, auto&& fn) {
        uint32_t run = sn;
        for_each_tile(pass, [&](int kt) {
          const uint32_t cs = run++;
          if (PAIR) fn(kt, 2u * cs + (uint32_t)grp);   // every tile, for this group's query tile
          else if ((cs & 1u) == (uint32_t)grp) fn(kt, cs);
        });
        sn = run;
      };

      if (MODE == ENTMAX) {
        const float c1 = p.scale * (p.alpha - 1.f);
        const float e = 1.f / (p.alpha - 1.f);
        // Row-max pass with streaming candidates.
        //
        // tau never drops below max - 1, and threads that have seen some of a row's scores can do
        // better.  With f(t) = sum_j [X_j - t]_+^e - 1 (convex, decreasing; its root is tau): leaving
        // entries out only lowers f, a tangent of a convex function lies below it, and a Newton step
        // from the left never passes the root.  So a root of "my candidates exactly + the tangents the
        // other three threads of the row published for theirs - 1", approached by Newton steps from
        // the left, is a lower bound of the row's threshold however stale the tangents are.
        // While it looks for the row maximum, every row thread keeps the scores of its columns that lie
        // above the best lower bound known for the row in kStageSlots private shared-memory slots; one
        // candidate costs a predicated shared-memory store and a predicated pointer bump.  After every
        // 8 scores a warp whose fullest lane has fewer than 8 free slots left tightens: each lane takes
        // Newton steps as above, publishes its tangent and the new bound, and drops the candidates at
        // or below it.  On a long Gaussian row the bound closes in on the threshold after a few tiles
        // and little more than the final support (a fraction of a percent of the row) is ever kept.
        // At the end of the pass the union of the four threads' candidates contains the row's support,
        // and the threshold is iterated to convergence on those few values: no further score
        // products, no key tile read again.  A tile is marked for the last pass iff a candidate was
        // taken from it.  If some lane cannot get down to kStageSlots - 8 candidates (wide supports:
        // alpha near 1, tiny scores), the CTA falls back to threshold passes over recomputed score
        // tiles, which mark tiles by their distance from the running maximum instead.
        float mrow = -INFINITY;
        uint32_t mark_bits = 0;
        int mark_word = 0;
        auto publish_marks = [&]() {
          const uint32_t any = __reduce_or_sync(0xffffffffu, mark_bits);
          if (any != 0u && lane == 0) atomicOr(&sh.act_next[mark_word], any);
          mark_bits = 0;
        };
        // (uniform over the CTA here, over the warp once a lane has run out of slots)
        // Which way by default: keeping candidates costs about as much CUDA-core work per score as one
        // threshold pass (three issue slots per score for the predicated store and pointer bump, plus the
        // tightening calls).  alpha = 2 pays that once instead of five or six Newton passes; alpha = 1.5,
        // whose tail-model first step gets by with three passes, comes out slightly behind and keeps the
        // passes unless the caller asks for candidates (the host side picks the kernel variant).
        bool lovf = !LISTS || p.niter <= 0;
        float* const stage_t = reinterpret_cast<float*>(stage) + tid;  // slot x of this thread: stage_t[x * 512]
        const uint32_t sa0 = smem_u32(stage_t);
        uint32_t sa = sa0;
        float tlb = -INFINITY;   // this thread's lower bound of the row threshold, (alpha-1)*score units
        uint32_t ntile = 0;      // tiles this thread has worked on
        volatile float* rlb = &sh.rlb[0][0];
        volatile float* rmx = &sh.rmax[0][0];
        // steps: Newton steps to take; keep_if: compact only if more than this many candidates are held
        auto tighten = [&](int steps, int keep_if) {
          const float blb = fmaxf(fmaxf(rlb[row], rlb[128 + row]), fmaxf(rlb[256 + row], rlb[384 + row]));
          const float msh_x = fmaxf(fmaxf(rmx[row], rmx[128 + row]), fmaxf(rmx[256 + row], rmx[384 + row])) * c1;
          const TightenResult tr = tighten_candidates<KIND>(&sh, stage_t, (int)((sa - sa0) >> 11), fmaxf(msh_x - 1.f, blb),
                                                            c1, e, quad, row, steps, keep_if);
          tlb = tr.bound;
          sa = sa0 + (uint32_t)max(tr.kept, 0) * 2048u;
          if (__any_sync(0xffffffffu, tr.kept < 0)) lovf = true;   // the spill pool is full
        };
        const float inv_c1 = 1.f / c1;
        for_my_tiles(0, [&](int kt, uint32_t cs) {
          const uint32_t buf = cs & 3;
          if ((kt >> 5) != mark_word) { publish_marks(); mark_word = kt >> 5; }
          mbar_wait(&sh.s_full[buf], (cs >> 2) & 1, abort_flag, status, 30);
          __syncwarp();
          tc_fence_after_sync();
          uint32_t r[64];
          tmem_ld64_sync(tgrp + buf * 128 + c0, r);
          tc_fence_before_sync();
          __syncwarp();   // every lane holds its scores: one arrival per warp
          if (lane == 0) mbar_arrive(&sh.s_free[buf]);
          if (kt * 128 + 127 > tile_jlim) {
            const int climit = jlim - kt * 128 - c0;
#pragma unroll
            for (int x = 0; x < 64; ++x)
              if (x > climit) r[x] = 0xff800000u;   // -inf
          }
          float m0 = -INFINITY, m1 = -INFINITY;
#pragma unroll
          for (int x = 0; x < 64; x += 2) {
            m0 = fmaxf(m0, __uint_as_float(r[x]));
            m1 = fmaxf(m1, __uint_as_float(r[x + 1]));
          }
          const float tm = fmaxf(m0, m1);
          mrow = fmaxf(mrow, tm);
          float msh = mrow;   // largest score any of the row's four threads has seen (exchanged only while
                              // candidates are kept: the filter gains from it, the tile marks hardly do)
          if (LISTS && !lovf) {
            rmx[quad * 128 + row] = mrow;
            msh = fmaxf(fmaxf(rmx[row], rmx[128 + row]), fmaxf(rmx[256 + row], rmx[384 + row]));
          }
          const bool near_max = tm > -INFINITY && (msh - tm) * c1 < 1.f;
          bool took = false;
          if (LISTS && !lovf) {
            // raw-score form of the row's best lower bound; masked entries are -inf and never pass
            const float blb = fmaxf(fmaxf(rlb[row], rlb[128 + row]), fmaxf(rlb[256 + row], rlb[384 + row]));
            const float thr = fmaxf(msh - inv_c1, blb * inv_c1);
#pragma unroll
            for (int x0 = 0; x0 < 64; x0 += 8) {
              if (lovf) break;   // (a lane ran out of slots: nothing more is staged)
              const uint32_t sa_in = sa;
#pragma unroll
              for (int x = x0; x < x0 + 8; ++x)
                asm volatile(
                    "{\n\t.reg .pred p;\n\t"
                    "setp.gt.f32 p, %1, %2;\n\t"
                    "@p st.shared.f32 [%0], %1;\n\t"
                    "@p add.u32 %0, %0, 2048;\n\t}"
                    : "+r"(sa)
                    : "f"(__uint_as_float(r[x])), "f"(thr)
                    : "memory");
              took |= sa != sa_in;
              if (__any_sync(0xffffffffu, sa - sa0 > (uint32_t)(kStageSlots - 8) * 2048u)) {
                tighten(3, 0);
              }
            }
          }
          // One Newton step at the end of a tile keeps the published tangents fresh and the bound close to
          // the threshold of what the row has shown so far; the bound moves less and less, so the steps
          // thin out: after the thread's tiles 1-4, then 6, 8, 12, 16, 24, 32, ...
          if (LISTS && !lovf) {
            ++ntile;
            const uint32_t third = ntile / 3u;
            const bool due = ntile <= 4u || (ntile & (ntile - 1u)) == 0u || (third * 3u == ntile && (third & (third - 1u)) == 0u);
            if (due) {
              tighten(1, 8);
            }
          }
          mark_bits |= (((!LISTS || lovf) ? near_max : took) ? 1u : 0u) << (kt & 31);
        });
        publish_marks();
        sh.part[quad][0][row] = mrow;
        sh.part[quad][1][row] = tlb;
        named_bar_sync(1, kFwdRowThreads);
        // (two-tile form: a row belongs to the two threads of one group)
        float m = PAIR ? fmaxf(sh.part[2 * grp][0][row], sh.part[2 * grp + 1][0][row])
                       : fmaxf(fmaxf(sh.part[0][0][row], sh.part[1][0][row]), fmaxf(sh.part[2][0][row], sh.part[3][0][row]));
        const float row_lb = PAIR ? fmaxf(sh.part[2 * grp][1][row], sh.part[2 * grp + 1][1][row])
                                  : fmaxf(fmaxf(sh.part[0][1][row], sh.part[1][1][row]), fmaxf(sh.part[2][1][row], sh.part[3][1][row]));
        if (warp == 0) {
          // tiles of the next pass (all of them if nothing was marked: non-finite scores)
          const int lo_t = lane * 32;
          const uint32_t full = nkt >= lo_t + 32 ? 0xffffffffu : (nkt > lo_t ? (1u << (nkt - lo_t)) - 1u : 0u);
          uint32_t nx = ((volatile uint32_t*)sh.act_next)[lane];
          if (!__any_sync(0xffffffffu, nx != 0u)) nx = full;
          sh.act[1][lane] = nx;
          sh.act_next[lane] = 0u;
        }
        const bool all_fit = named_bar_and(2, kFwdRowThreads, !lovf);
        const bool use_list = LISTS && all_fit;
        m = live ? m * c1 : 0.f;
        const float n = (float)(jlim + 1);
        float ts = -1.f, lo = -1.f, hi = live ? -exp2f(-(p.alpha - 1.f) * log2f(fmaxf(n, 1.f))) : -1.f;
        bool done = !live || n <= 1.f;
        // One update of this row's threshold from the three sums over its support; returns true when
        // the threshold fell by more than rounding (tile skipping relies on it not falling).
        auto update_tau = [&](float sum0, float sum1, float sum2v, int it, float tol_halley, float tol_newton,
                              float tol_bisect) {
          bool regular;
          float t = tau_update(ts, sum0, sum1, sum2v, e, lo, hi, &regular);
          if (KIND == 0 && it == 0 && !(p.flags & FLA_FLAG_PLAIN_FIRST_STEP)) {
            // first step of a row: the tail-model step where the moments admit it
            const float jump = gpd_first_step(sum0, sum1, sum2v);
            if (jump > 0.f && ts + jump > t && ts + jump <= hi) { t = ts + jump; regular = false; }
          }
          const float tol = regular ? (e >= 2.f ? tol_halley : tol_newton) : tol_bisect;
          // quadratic / cubic convergence: once a step is this small the next one is far below
          // fp32 resolution; the second term covers rows whose |tau| is too large to resolve it
          if (fabsf(t - ts) <= fmaxf(tol, 4e-7f * fabsf(m))) done = true;
          if (t >= ts) { ts = t; return false; }
          if (ts - t > 2e-6f * fmaxf(1.f, fabsf(m))) { ts = t; return true; }
          return false;
        };
        if (use_list) {
          // ---- threshold iteration on the candidates: the producer and the issuers go straight to the
          // last pass (tiles a candidate was taken from) while the row threads iterate
          signal_pass(false);
          rpass = 1;
          if (tid == 0 && status) atomicAdd(status + 6, 1);
          const int n_st = (int)((sa - sa0) >> 11);
          const int npool = min(*(volatile int*)&sh.npool, kPoolSize);
          // start from the row's best lower bound (still left of the root)
          if (live && row_lb - m > ts) { ts = fminf(row_lb - m, hi); lo = ts; }
          for (int it = 0; it < p.niter; ++it) {
            float a0 = 0.f, a1 = 0.f, a2 = 0.f;
            const float noff = -(m + ts);   // d = X - tau with X = s*c1
            for (int j = 0; j < n_st; ++j) {
              const float d = fmaf(stage_t[j * kFwdRowThreads], c1, noff);
              if (KIND == 0) {
                const float ee = __saturatef(d);   // d <= 1 on the whole bracket
                a0 = fmaf(ee, ee, a0); a1 += ee; a2 += d > 0.f ? 1.f : 0.f;
              } else if (KIND == 1) {
                a0 += fmaxf(d, 0.f); a1 += d > 0.f ? 1.f : 0.f;
              } else if (d > 0.f) {
                float pw, u;
                p_and_u<2>(d, e, pw, u);
                a0 += pw; a1 += u; a2 += __fdividef(u, d);
              }
            }
            // spilled candidates: pool entry i is summed by thread i mod 4 of its row
            for (int i2 = quad; i2 < npool; i2 += 4) {
              const float2 pe = sh.pool[i2];
              if (__float_as_int(pe.y) == row) {
                const float d = fmaf(pe.x, c1, noff);
                if (KIND == 0) {
                  const float ee = __saturatef(d);
                  a0 = fmaf(ee, ee, a0); a1 += ee; a2 += d > 0.f ? 1.f : 0.f;
                } else if (KIND == 1) {
                  a0 += fmaxf(d, 0.f); a1 += d > 0.f ? 1.f : 0.f;
                } else if (d > 0.f) {
                  float pw, u;
                  p_and_u<2>(d, e, pw, u);
                  a0 += pw; a1 += u; a2 += __fdividef(u, d);
                }
              }
            }
            sh.part[quad][0][row] = a0;
            sh.part[quad][1][row] = a1;
            sh.part[quad][2][row] = a2;
            named_bar_sync(1, kFwdRowThreads);
            if (!done) {
              const float sum0 = (sh.part[0][0][row] + sh.part[1][0][row]) + (sh.part[2][0][row] + sh.part[3][0][row]);
              const float sum1 = (sh.part[0][1][row] + sh.part[1][1][row]) + (sh.part[2][1][row] + sh.part[3][1][row]);
              const float sum2v = (sh.part[0][2][row] + sh.part[1][2][row]) + (sh.part[2][2][row] + sh.part[3][2][row]);
              // an iteration costs a few hundred cycles here, not a pass over the keys: converge.  (No
              // tail-model first step: the candidates below the lower bound are gone, and with them the
              // moments at max - 1 that step is fitted to.)
              update_tau(sum0, sum1, sum2v, it + 1, kListTolHalley, kListTolNewton, kListTol);
            }
            // (the barrier also orders this iteration's reads of the partial sums before the next writes)
            if (named_bar_and(2, kFwdRowThreads, done || *abort_flag != 0)) break;
          }
          // Canonical finish (alpha = 1.5 and 2).  Which candidates a thread still holds, the point the
          // iteration started from and the order of the pool depend on how the warps happened to interleave,
          // so the converged threshold differs from run to run in its last bits -- enough to flip an entry
          // sitting on the threshold and, with it, a whole row of gradients (the entmax Jacobian jumps where
          // the support changes).  The iteration is therefore only trusted to identify the support; the
          // threshold is then recomputed from it in closed form, from sums formed as integers (order does
          // not matter) of z = X - max rounded to 2^-24:  alpha = 2: tau = (sum z - 1) / n;  alpha = 1.5:
          // the smaller root of  n tau^2 - 2 tau sum z + sum z^2 - 1 = 0.  Same support, same bits.
          if (KIND != 2 && !*abort_flag) {
            long long zs1 = 0, zs2 = 0;
            int zn = 0;
            const float noff = -(m + ts);
            auto take = [&](float sv) {
              if (fmaf(sv, c1, noff) > 0.f) {
                const long long zi = __float2ll_rn(fmaf(sv, c1, -m) * 16777216.f);
                zs1 += zi;
                if (KIND == 0) zs2 += zi * zi;
                ++zn;
              }
            };
            for (int j = 0; j < n_st; ++j) take(stage_t[j * kFwdRowThreads]);
            for (int i2 = quad; i2 < npool; i2 += 4) {
              const float2 pe = sh.pool[i2];
              if (__float_as_int(pe.y) == row) take(pe.x);
            }
            // the four threads of a row exchange through their own first candidate slots (all read by now)
            uint32_t* const xs = reinterpret_cast<uint32_t*>(stage_t);
            xs[0] = (uint32_t)zn;
            xs[1 * kFwdRowThreads] = (uint32_t)(unsigned long long)zs1;
            xs[2 * kFwdRowThreads] = (uint32_t)((unsigned long long)zs1 >> 32);
            xs[3 * kFwdRowThreads] = (uint32_t)(unsigned long long)zs2;
            xs[4 * kFwdRowThreads] = (uint32_t)((unsigned long long)zs2 >> 32);
            named_bar_sync(1, kFwdRowThreads);
            long long t1 = 0, t2 = 0;
            int tn = 0;
#pragma unroll
            for (int qq = 0; qq < 4; ++qq) {
              // thread `qq` of this row: warp (row / 32) + 4 (qq / 2) + 8 (qq % 2), same lane
              const uint32_t* xo = reinterpret_cast<const uint32_t*>(stage) + (((row >> 5) + 4 * (qq >> 1) + 8 * (qq & 1)) * 32 + (row & 31));
              tn += (int)xo[0];
              t1 += (long long)((unsigned long long)xo[1 * kFwdRowThreads] | ((unsigned long long)xo[2 * kFwdRowThreads] << 32));
              t2 += (long long)((unsigned long long)xo[3 * kFwdRowThreads] | ((unsigned long long)xo[4 * kFwdRowThreads] << 32));
            }
            if (live && tn > 0) {
              const double zsum = (double)t1 * (1.0 / 16777216.0), nd = (double)tn;
              double zt;
              if (KIND == 1) {
                zt = (zsum - 1.0) / nd;
              } else {
                const double zsq = (double)t2 * (1.0 / 16777216.0 / 16777216.0);
                const double disc = zsum * zsum - nd * (zsq - 1.0);
                zt = (zsum - sqrt(fmax(disc, 0.0))) / nd;
              }
              // (taken only if it agrees with the iteration: it cannot differ by more than rounding unless
              // an entry sat on the threshold or the iteration was cut short by niter)
              if (fabs(zt - (double)ts) <= 1e-4) ts = (float)zt;
            }
          }
        } else {
          if (tid == 0 && status) atomicAdd(status + 7, 1);
          bool cont = p.niter > 0;
          signal_pass(cont);
          rpass = 1;
          for (int it = 0; cont; ++it) {
            float a0 = 0.f, a1 = 0.f, a2 = 0.f, b0 = 0.f, b1 = 0.f, b2 = 0.f;
            const float off = m + ts;   // d = X - tau with X = s*c1
            // tiles with an entry above tau, collected per 32-tile word and published once per word
            uint32_t hit_bits = 0;
            int hit_word = 0;
            auto publish_hits = [&]() {
              const uint32_t any = __reduce_or_sync(0xffffffffu, hit_bits);
              if (any != 0u && lane == 0) atomicOr(&sh.act_next[hit_word], any);
              hit_bits = 0;
            };
            // The two groups take turns at the arithmetic: a group sums its tile while the other
            // one waits for its next score tile and loads it, so the floating-point pipe of a
            // scheduler serves two warps at a time instead of four in lockstep followed by none.
            // Barrier 4 + g is group g's "your turn"; the group owning the first tile of the pass
            // gets the first turn from the other one, and whoever did not sum last takes the
            // turn that is left over.
            const uint32_t first_grp = sn & 1u;
            int nact_pass = 0;
            for (int w = 0; w * 32 < nkt; ++w) nact_pass += __popc(((volatile uint32_t*)sh.act[rpass & 1u])[w]);
            // (general alpha: no turns.  Its arithmetic is a long dependent chain per entry on a divergent path, and
            // four warps per scheduler hide that latency better than two.)
            constexpr bool kTurns = KIND != 2 && !PAIR;   // (two-tile form: both groups sum at once)
            if (kTurns && (uint32_t)grp != first_grp) named_bar_arrive(4 + (int)first_grp, kFwdRowThreads);
            for_my_tiles(rpass, [&](int kt, uint32_t cs) {
              const uint32_t buf = cs & 3;
              bool hit = false;           // some entry of this tile lies above tau
              if ((kt >> 5) != hit_word) { publish_hits(); hit_word = kt >> 5; }
              mbar_wait(&sh.s_full[buf], (cs >> 2) & 1, abort_flag, status, 31);
              __syncwarp();
              tc_fence_after_sync();
              // this thread's half row into registers, buffer handed back at once: the next product
              // into this buffer runs while the row is summed
              uint32_t r[64];
              tmem_ld64_sync(tgrp + buf * 128 + c0, r);
              tc_fence_before_sync();
              // the token is zero; adding it makes every sum below depend on the arrive, so the
              // buffer is handed back before the arithmetic instead of after it
              __syncwarp();   // every lane holds its scores: one arrival per warp
              float noff = __uint_as_float(lane == 0 ? mbar_arrive_token(&sh.s_free[buf]) : 0u) - off;
              const bool need_mask = kt * 128 + 127 > tile_jlim;
              if (need_mask) {   // diagonal / sequence end: masked entries contribute nothing
                const int climit = jlim - kt * 128 - c0;
  #pragma unroll
                for (int x = 0; x < 64; ++x)
                  if (x > climit) r[x] = 0xff800000u;   // -inf
              }
              if (kTurns) noff += __uint_as_float(named_bar_sync_token(4 + grp, kFwdRowThreads));   // my turn
              if (KIND == 0) {
                // alpha = 1.5: d <= 1 on the whole bracket, so one saturating fma yields max(d, 0)
                // (and 0 for a masked entry); sums kept as packed pairs
                uint64_t s0 = pack2(0.f, 0.f), s1 = s0, s2 = s0;
  #pragma unroll
                for (int x = 0; x < 64; x += 2) {
                  const float e0 = __saturatef(fmaf(__uint_as_float(r[x]), c1, noff));
                  const float e1 = __saturatef(fmaf(__uint_as_float(r[x + 1]), c1, noff));
                  const uint64_t ee = pack2(e0, e1);
                  s0 = fma2(ee, ee, s0);
                  s1 = add2(s1, ee);
                  s2 = add2(s2, pack2(e0 > 0.f ? 1.f : 0.f, e1 > 0.f ? 1.f : 0.f));
                }
                const float cnt = sum2(s2);
                a0 += sum2(s0); a1 += sum2(s1); a2 += cnt;
                hit = cnt > 0.f;
              } else {
                auto chunk_sums = [&](const uint32_t* rc) {
  #pragma unroll
                  for (int x = 0; x < 32; x += 2) {
                    const float d0 = fmaf(__uint_as_float(rc[x]), c1, noff);
                    const float d1 = fmaf(__uint_as_float(rc[x + 1]), c1, noff);
                    hit |= (d0 > 0.f) | (d1 > 0.f);
                    if (KIND == 0) {
                      const float e0 = fmaxf(d0, 0.f), e1 = fmaxf(d1, 0.f);
                      a0 = fmaf(e0, e0, a0); a1 += e0; a2 += d0 > 0.f ? 1.f : 0.f;
                      b0 = fmaf(e1, e1, b0); b1 += e1; b2 += d1 > 0.f ? 1.f : 0.f;
                    } else if (KIND == 1) {
                      a0 += fmaxf(d0, 0.f); a1 += d0 > 0.f ? 1.f : 0.f;
                      b0 += fmaxf(d1, 0.f); b1 += d1 > 0.f ? 1.f : 0.f;
                    } else {
                      if (d0 > 0.f) { float pw, u; p_and_u<2>(d0, e, pw, u); a0 += pw; a1 += u; a2 += __fdividef(u, d0); }
                      if (d1 > 0.f) { float pw, u; p_and_u<2>(d1, e, pw, u); b0 += pw; b1 += u; b2 += __fdividef(u, d1); }
                    }
                  }
                };
                chunk_sums(r);
                chunk_sums(r + 32);
              }
              // hand the turn over once the sums are done (the sums feed the barrier's memory clobber)
              if (kTurns) named_bar_arrive_after(4 + (grp ^ 1), kFwdRowThreads, a0 + b0, a1 + b1, a2 + b2);
              hit_bits |= (hit ? 1u : 0u) << (kt & 31);
            });
            {
              // the group that did not sum last consumes the turn that is left over
              const uint32_t last_grp = (first_grp + (uint32_t)nact_pass + 1u) & 1u;
              if (kTurns && (nact_pass > 0 ? (uint32_t)grp != last_grp : (uint32_t)grp == first_grp)) named_bar_sync(4 + grp, kFwdRowThreads);
            }
            publish_hits();
            sh.part[quad][0][row] = a0 + b0;
            sh.part[quad][1][row] = a1 + b1;
            sh.part[quad][2][row] = a2 + b2;
            named_bar_sync(1, kFwdRowThreads);
            if (!done) {
              const float sum0 = PAIR ? sh.part[2 * grp][0][row] + sh.part[2 * grp + 1][0][row]
                                      : (sh.part[0][0][row] + sh.part[1][0][row]) + (sh.part[2][0][row] + sh.part[3][0][row]);
              const float sum1 = PAIR ? sh.part[2 * grp][1][row] + sh.part[2 * grp + 1][1][row]
                                      : (sh.part[0][1][row] + sh.part[1][1][row]) + (sh.part[2][1][row] + sh.part[3][1][row]);
              const float sum2v = PAIR ? sh.part[2 * grp][2][row] + sh.part[2 * grp + 1][2][row]
                                       : (sh.part[0][2][row] + sh.part[1][2][row]) + (sh.part[2][2][row] + sh.part[3][2][row]);
              // Tile skipping relies on tau not falling.  A fall within rounding is dropped; a real
              // one (after a first step that overshot, or a bisection) makes the next pass visit the
              // tiles of the first threshold pass again: tau never leaves the bracket, whose lower
              // end is where that pass evaluated.
              if (update_tau(sum0, sum1, sum2v, it, kTauTolHalley, kTauTolNewton, kTauTol)) *(volatile int*)&sh.force_all = 1;
            }
            const bool all_done = named_bar_and(2, kFwdRowThreads, done);
            cont = !all_done && (it + 1 < p.niter) && !*abort_flag;
            if (warp == 0) {
              // tiles of the next pass: those in which some row found an entry above its tau
              const int lo_t = lane * 32;
              const uint32_t full = nkt >= lo_t + 32 ? 0xffffffffu : (nkt > lo_t ? (1u << (nkt - lo_t)) - 1u : 0u);
              uint32_t nx = ((volatile uint32_t*)sh.act_next)[lane];
              const bool none = !__any_sync(0xffffffffu, nx != 0u);   // only with non-finite scores
              if (it == 0) sh.act_base[lane] = none ? full : nx;
              if (none) nx = full;
              if (*(volatile int*)&sh.force_all) nx = sh.act_base[lane];   // some tau fell in this step
              sh.act[(rpass + 1u) & 1u][lane] = nx;
              sh.act_next[lane] = 0u;
              __syncwarp();
              if (lane == 0) *(volatile int*)&sh.force_all = 0;
            }
            named_bar_sync(3, kFwdRowThreads);
            ++rpass;
            signal_pass(cont);
          }
        }
        rstat = m + ts;
      } else {
        // Lazy Attention: online log-sum-exp in the log2 domain, one partial (m, l) per thread
        const float sl2 = p.scale * kLog2e;
        float m = -INFINITY, l = 0.f;
        for_my_tiles(0, [&](int kt, uint32_t cs) {
          const uint32_t buf = cs & 3;
          mbar_wait(&sh.s_full[buf], (cs >> 2) & 1, abort_flag, status, 32);
          __syncwarp();
          tc_fence_after_sync();
          const bool need_mask = kt * 128 + 127 > tile_jlim;
          const int climit = jlim - kt * 128 - c0;
          const bool in_window = row0 - kt * 128 - 127 < p.window;
          // 32 columns at a time (small loop body); the running (m, l) is rescaled per chunk
#pragma unroll 1
          for (int ch = 0; ch < 2; ++ch) {
            uint32_t r[32];
            tmem_ld32_sync(tgrp + buf * 128 + c0 + ch * 32, r);
            if (ch == 1) {
              tc_fence_before_sync();
              __syncwarp();
              if (lane == 0) mbar_arrive(&sh.s_free[buf]);
            }
            float tmax = -INFINITY;
            if (!in_window && !need_mask) {
              // interior tile (no bias, no masked entry): the maximum is taken over the raw scores (the scale is
              // positive), the scale is folded into the exponent's fused multiply-add, pairs go through packed
              // f32x2 operations
              float rmax = -INFINITY;
#pragma unroll
              for (int x = 0; x < 32; ++x) rmax = fmaxf(rmax, __uint_as_float(r[x]));
              const float mn = fmaxf(m, rmax * sl2);
              if (mn > -INFINITY) {
                const uint64_t s2 = pack2(sl2, sl2), nm = pack2(-mn, -mn);
                uint64_t acc = pack2(0.f, 0.f);
#pragma unroll
                for (int x = 0; x < 32; x += 2) {
                  float x0, x1;
                  unpack2(fma2(pack2(__uint_as_float(r[x]), __uint_as_float(r[x + 1])), s2, nm), x0, x1);
                  acc = add2(acc, pack2(fast_exp2(x0), fast_exp2(x1)));
                }
                l = l * fast_exp2(m - mn) + sum2(acc);
                m = mn;
              }
              continue;
            } else
#pragma unroll
            for (int x = 0; x < 32; ++x) {
              float v = __uint_as_float(r[x]) * sl2;
              if (in_window) {
                const int dist = i - (kt * 128 + c0 + ch * 32 + x);
                if (dist >= 0 && dist < p.window) v = fmaf(__ldg(p.bias + (int64_t)h * p.bias_stride + dist), kLog2e, v);
              }
              if (need_mask && ch * 32 + x > climit) v = -INFINITY;
              r[x] = __float_as_uint(v);
              tmax = fmaxf(tmax, v);
            }
            const float mn = fmaxf(m, tmax);
            if (mn > -INFINITY) {
              float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
              for (int x = 0; x < 32; x += 2) {
                acc0 += fast_exp2(__uint_as_float(r[x]) - mn);
                acc1 += fast_exp2(__uint_as_float(r[x + 1]) - mn);
              }
              l = l * fast_exp2(m - mn) + acc0 + acc1;
              m = mn;
            }
          }
        });
        sh.part[quad][0][row] = m;
        sh.part[quad][1][row] = l;
        named_bar_sync(1, kFwdRowThreads);
        {
          float mm = -INFINITY;
#pragma unroll
          for (int qd = 0; qd < 4; ++qd) mm = fmaxf(mm, sh.part[qd][0][row]);
          float ll = 0.f;
#pragma unroll
          for (int qd = 0; qd < 4; ++qd) {
            const float mq = sh.part[qd][0][row];
            if (mq > -INFINITY) ll += sh.part[qd][1][row] * fast_exp2(mq - mm);
          }
          rstat = (live && ll > 0.f) ? mm + log2f(ll) : 0.f;
        }
        named_bar_sync(2, kFwdRowThreads);
        signal_pass(false);
        rpass = 1;
      }

      // ---- last pass ------------------------------------------------------------------------------
      // One-tile form: the two groups take alternate key tiles of the one query tile.  Two-tile form: group g works
      // on its own query tile for every key tile and writes the probabilities over the scores it read them from
      // (score buffer g; accumulator g), see the issuers.
      {
      constexpr int sub = 0;
      const int i_s = i;
      const bool live_s = live;
      const int jlim_s = jlim;
      const int tile_jlim_s = tile_jlim;
      const float rstat_s = rstat;
      const uint32_t use0 = 0;
      uint32_t* const my_mask = PAIR && grp == 1 ? reinterpret_cast<uint32_t*>(stage) : sh.mask_words;   // (two-tile form: the second
                                                                  // tile's block-mask words live behind the ring)
      // ---- last pass: probabilities into tensor memory --------------------------------------
      // S(t) lands in score buffer t & 1; the probabilities go to a buffer of their own (64 columns
      // behind the output accumulator), so the next score product into the same score buffer
      // needs only these threads to have read it, not the P.V product to have finished.
      const float c1 = p.scale * (MODE == ENTMAX ? (p.alpha - 1.f) : kLog2e);
      const float e = MODE == ENTMAX ? 1.f / (p.alpha - 1.f) : 0.f;
      const float tau_row = MODE == LAZY ? p.tau_h[h] / (float)(i_s + 1) : 0.f;
      const uint32_t sbase = tgrp + grp * 128 + c0;                 // my half of score buffer grp
      const uint32_t pbase = tgrp + kProbCol + grp * 64 + half * 32;   // my half of probability buffer grp
      uint32_t u_run = 0;
      for_each_tile(rpass, [&](int kt) {
        const uint32_t u = u_run++;
        if (!PAIR && (u & 1u) != (uint32_t)grp) return;
        const uint32_t use = PAIR ? u : use0 + (u >> 1);    // of the buffers of this group (they complete once per tile of its)
        mbar_wait(&sh.f_full[grp], use & 1u, abort_flag, status, 33);
        // the P.V product that last read this probability buffer must be done (two-tile form: the score product
        // waited for it already)
        if (!PAIR && use >= 1u) mbar_wait(&sh.pv_done[grp], (use - 1u) & 1u, abort_flag, status, 36);
        __syncwarp();
        tc_fence_after_sync();
        const bool need_mask = kt * 128 + 127 > tile_jlim_s;
        const int climit = jlim_s - kt * 128 - c0;
        const bool in_window = MODE == LAZY && (row0 - kt * 128 - 127 < p.window);
        uint32_t nz = 0;
#pragma unroll 1
        for (int ch = 0; ch < 2; ++ch) {
          uint32_t r[32], pk[16];
          tmem_ld32_sync(sbase + ch * 32, r);
          if (MODE == ENTMAX && KIND == 0 && !need_mask) {
            // alpha = 1.5, no masked entry: P = max(x, 0)^2 with the clamp folded into the fma
#pragma unroll
            for (int x = 0; x < 32; x += 2) {
              const float e0 = __saturatef(fmaf(__uint_as_float(r[x]), c1, -rstat_s));
              const float e1 = __saturatef(fmaf(__uint_as_float(r[x + 1]), c1, -rstat_s));
              pk[x >> 1] = pack16<FMT>(e0 * e0, e1 * e1);
              nz |= pk[x >> 1];
            }
          } else if (MODE == LAZY && !need_mask && !in_window) {
            // interior tile: A = max(exp2(x - lse) + tau_h/(i_s+1), 0), straight-line
#pragma unroll
            for (int x = 0; x < 32; x += 2) {
              const float t0 = fast_exp2(fmaf(__uint_as_float(r[x]), c1, -rstat_s)) + tau_row;
              const float t1 = fast_exp2(fmaf(__uint_as_float(r[x + 1]), c1, -rstat_s)) + tau_row;
              pk[x >> 1] = pack16<FMT>(fmaxf(t0, 0.f), fmaxf(t1, 0.f));
              nz |= pk[x >> 1];
            }
          } else {
#pragma unroll
            for (int x = 0; x < 32; x += 2) {
              float pv[2];
#pragma unroll
              for (int y = 0; y < 2; ++y) {
                const int c = ch * 32 + x + y;
                const float sc = __uint_as_float(r[x + y]);
                const bool valid = !need_mask || c <= climit;
                float pw = 0.f;
                if (MODE == ENTMAX) {
                  const float d = fmaf(sc, c1, -rstat_s);
                  if (valid && d > 0.f) pw = pow_e<KIND>(d, e);
                } else {
                  float v = sc * c1;
                  if (in_window) {
                    const int dist = i_s - (kt * 128 + c0 + c);
                    if (dist >= 0 && dist < p.window) v = fmaf(__ldg(p.bias + (int64_t)h * p.bias_stride + dist), kLog2e, v);
                  }
                  const float t = fast_exp2(v - rstat_s) + tau_row;
                  if (valid && t > 0.f) pw = t;
                }
                pv[y] = pw;
              }
              pk[x >> 1] = pack16<FMT>(pv[0], pv[1]);
              nz |= pk[x >> 1];
            }
          }
          tmem_st16(PAIR ? sbase + ch * 32 : pbase + ch * 16, pk);
        }
        tmem_st_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&sh.p_full[grp]);
        if (MODE == ENTMAX && p.block_mask != nullptr) {
          // key block (64 keys) 2 kt + half holds a non-zero probability for some row of this warp
          if (__any_sync(0xffffffffu, nz != 0) && lane == 0) {
            const int j = 2 * kt + half;
            atomicOr(&my_mask[j >> 5], 1u << (j & 31));
          }
        }
      });

      // ---- epilogue: each of the four (two-tile form: two) threads of a row stores its share of the output columns
      mbar_wait(&sh.o_full, 0, abort_flag, status, 34);
      __syncwarp();
      tc_fence_after_sync();
      const bool in_range = i_s < L;
      uint8_t* orow = (uint8_t*)p.o.ptr + 2 * ((int64_t)b * p.o.s[0] + (int64_t)h * p.o.s[1] + (int64_t)i_s * p.o.s[2]);
      // columns [col0, col0 + 32 nld) of the accumulator: a quarter of the row, or half of it
      const int nld = PAIR ? D / 64 : (quad < D / 32 ? 1 : 0);
      const int col0 = PAIR ? half * (D / 2) : quad * 32;
      const uint32_t acc = PAIR ? tmem + 256 + grp * 128 : tmem_o;
      for (int part = 0; part < nld; ++part) {
        uint32_t r[32];
        tmem_ld32_sync(acc + lane_base + col0 + part * 32, r);
        if (in_range) {
#pragma unroll
          for (int x = 0; x < 32; x += 8) {
            uint4 w;
            w.x = live_s ? pack16<FMT>(__uint_as_float(r[x]), __uint_as_float(r[x + 1])) : 0u;
            w.y = live_s ? pack16<FMT>(__uint_as_float(r[x + 2]), __uint_as_float(r[x + 3])) : 0u;
            w.z = live_s ? pack16<FMT>(__uint_as_float(r[x + 4]), __uint_as_float(r[x + 5])) : 0u;
            w.w = live_s ? pack16<FMT>(__uint_as_float(r[x + 6]), __uint_as_float(r[x + 7])) : 0u;
            *(uint4*)(orow + (col0 + part * 32 + x) * 2) = w;
          }
        }
      }
      if (in_range && (PAIR ? half == 0 : quad == 0)) {
        if (MODE == ENTMAX) p.tau[bhl + i_s] = live_s ? rstat_s : 0.f;
        else p.lse[bhl + i_s] = live_s ? rstat_s : 0.f;
      }
      named_bar_sync(1, kFwdRowThreads);
      if (MODE == ENTMAX && p.block_mask != nullptr && tid < p.mask_words) {
        p.block_mask[((int64_t)bh * nmt + mt + sub) * p.mask_words + tid] = sh.mask_words[tid];
        if (PAIR && mt + 1 < nmt)
          p.block_mask[((int64_t)bh * nmt + mt + 1) * p.mask_words + tid] = reinterpret_cast<uint32_t*>(stage)[tid];
      }
      }
    } else if (i < L) {
      // the whole tile is padding: zeros (two-tile form: a row has the two threads of one group, half a row each)
      uint8_t* orow = (uint8_t*)p.o.ptr + 2 * ((int64_t)b * p.o.s[0] + (int64_t)h * p.o.s[1] + (int64_t)i * p.o.s[2]);
      if (PAIR) {
#pragma unroll
        for (int x = 0; x < D / 2; x += 8) *(uint4*)(orow + (half * (D / 2) + x) * 2) = make_uint4(0u, 0u, 0u, 0u);
        if (half == 0) p.tau[bhl + i] = 0.f;
      } else {
        if (quad < D / 32) {
#pragma unroll
          for (int x = 0; x < 32; x += 8) *(uint4*)(orow + (quad * 32 + x) * 2) = make_uint4(0u, 0u, 0u, 0u);
        }
        if (quad == 0) {
          if (MODE == ENTMAX) p.tau[bhl + i] = 0.f;
          else p.lse[bhl + i] = 0.f;
        }
      }
    }
    tc_fence_before_sync();
  }

  __syncthreads();
  if (*abort_flag) {  // leave time for copies still in flight before the shared memory is released
    for (int w = 0; w < 2000; ++w) __nanosleep(1000);
  }
  if (tid == 0) kernel_clock(status, 0, true);
  if (warp == kFwdProducerWarp) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, 512);
  }
}

}  // namespace tc
}  // namespace fla
