// Tensor-core backward of alpha-entmax attention and Lazy Attention: two warp-specialised
// kernels sharing the forward's building blocks (this file: dq_kernel and the shared helpers).
//
//   dq_kernel    one CTA per 128-row query tile.  Q and dO stay in shared memory, K tiles stream
//                through three slots (two for Lazy Attention) and V tiles through two, twice.  First sweep: S = Q.K^T and
//                dP = dO.V^T per key tile (two tiles in flight), row threads accumulate in fp32
//                the row scalar delta = sum_j U dP / sum_j U (entmax) or sum_j P M dP (lazy, plus
//                r = sum_j M dP for dtau); delta is also stored for dkdv_kernel.  Second sweep:
//                the same two products, row threads form dS = U (dP - delta) (entmax) or
//                P (M dP - delta) (lazy), write it back as a 16-bit A operand -> dQ += dS.K.
//                Lazy Attention also folds dS along its diagonals into dbias.
//   dkdv_kernel  lives in tc_bwd_kv.cuh.
//
// Replaces lazy_attention_triton.py:272-497 (dQ and dK/dV kernels) and the adasplash backward
// (source absent from the reference checkout); the first sweep of dq_kernel replaces the
// reference's pre-pass kernel lazy_attention_triton.py:180-270.  dkdv_kernel runs after
// dq_kernel on the same stream and reads the delta it stored.
#pragma once

#include "common.cuh"
#include "tc_fwd.cuh"
#include "tc_prims.cuh"

namespace fla {
namespace tc {

constexpr int kBwdThreads = 640;
constexpr int kBwdRowThreads = 512;   // warps 0-15, four threads per tile row
constexpr int kBwdRowWarps = 16;
constexpr int kBwdProducerWarp = 16;  // warps 17, 18 and 19 issue the products

constexpr int kBwdMaxTiles = 512;     // key tiles per row of the tile list: L <= 65536

struct BwdShared {
  uint64_t res_full, k_full[3], k_empty[3], v_full[2], v_empty[2];   // K and V slots are released separately
  uint64_t t_full[2], t_free[2], sweep_done;                           // first sweep
  uint64_t s_full, s_free, dp_full[2], ds_full[2], dq_done[2], acc_full;   // second sweep
  uint32_t tmem_base;
  int abort_flag;
  int nact;                 // number of key tiles this CTA visits
  uint16_t tiles[kBwdMaxTiles];   // their indices, ascending (every tile, or the ones the block mask marks)
};

// K tiles in flight.  A K tile is held from its copy until the dQ product of its tile has completed
// (S, the row threads and dQ in sequence), a V tile only until dP: with two K slots every K copy
// waited for the dQ product of the tile before the previous one and the tensor pipe idled for the
// copy's latency; a third slot takes that wait off the chain.  It fits next to the resident Q and dO
// tiles and two V slots (7 tiles = 224 KB at D = 128) only because this kernel keeps almost nothing
// else in shared memory: the Lazy variant's dbias sums go from the warps straight to the fixed-point
// accumulators in global memory (64 additions per warp and window tile, see the second sweep).
constexpr int kBwdKSlots = 3;

// Key tiles a query block has to visit: all of them, or -- with a block mask from the forward --
// those holding a non-zero probability (two 64-key mask bits per 128-key tile).  Run by one warp;
// returns the count (same value in every lane).
__device__ __forceinline__ int build_tile_list(uint16_t* tiles, int nkt, const uint32_t* mask_row, int lane) {
  int n = 0;
  for (int base = 0; base < nkt; base += 32) {
    const int kt = base + lane;
    bool on = kt < nkt;
    if (on && mask_row != nullptr) on = ((mask_row[(2 * kt) >> 5] >> ((2 * kt) & 31)) & 3u) != 0u;
    const uint32_t votes = __ballot_sync(0xffffffffu, on);
    if (on) tiles[n + __popc(votes & ((1u << lane) - 1u))] = (uint16_t)kt;
    n += __popc(votes);
  }
  return n;
}

// One score entry -> probability-like factors.
//   entmax: x = s*c1 - tau;  pv = P,  w = U            dS = w (dP - delta)
//   lazy:   x = s*c1 [+ bias] - lse2;  pv = A, w = Pn, m = [A > 0]   dS = w (m dP - delta)
template <int MODE, int KIND>
__device__ __forceinline__ void prob_terms(float x, float e, float tau_row, bool valid, float& pv, float& w,
                                           bool& m) {
  pv = 0.f;
  w = 0.f;
  m = false;
  if (MODE == ENTMAX) {
    if (valid && x > 0.f) { p_and_u<KIND>(x, e, pv, w); m = true; }
  } else {
    if (valid) {
      w = fast_exp2(x);
      const float t = w + tau_row;
      m = t > 0.f;
      pv = m ? t : 0.f;
    }
  }
}


// ------------------------------------------------------------------------------------------------
// Warps 0-15: row threads, four per query row (thread q of a row takes keys [32q, 32q+32) of every
// tile: sixteen warps keep the schedulers busy while others wait for a product, and the single S buffer of the
// second sweep is read out in half the time it took with eight); warp 16: copy producer; warps 17, 18, 19:
// issuers of S = Q.K^T, of dP = dO.V^T and of dQ += dS.K.  One thread per kind of product: a thread's waits, commits and loop run in sequence
// with its (blocking) issue, and a thread that waits for the operands of one product cannot issue
// another whose operands are ready (dQ of a tile would wait behind the K tile of the next one,
// which in turn waits for the ring slot that this very dQ product releases).
//
// Tensor-memory columns.  First sweep, tile g in slot j = g & 1: S at 256 j, dP at 256 j + 128.
// Second sweep: S at 0, dP of tile t at 128 + 128 (t & 1), dQ at 384.  dS overwrites dP as 16-bit
// pairs: thread q of a row writes columns [32q, 32q+16) of the buffer, inside the range it has already
// read, so the four never touch each other's input.
template <int MODE, int D, int FMT, int KIND>
__global__ void __launch_bounds__(kBwdThreads, 1)
dq_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
          const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do,
          const AttnParams p, int* status) {
  using Cfg = TileCfg<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align_1024(smem_raw);
  uint8_t* sQ = smem;
  uint8_t* sdO = smem + Cfg::kTileBytes;
  constexpr int NK = kBwdKSlots;
  uint8_t* ring = smem + 2 * Cfg::kTileBytes;  // NK slots for K tiles, then two for V tiles
  auto k_slot = [](int g) { return g % NK; };
  auto k_phase = [](int g) { return (uint32_t)((g / NK) & 1); };
  __shared__ BwdShared sh;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool causal = (MODE == LAZY) ? true : (p.causal != 0);
  const int L = p.L;
  const int nmt = (L + 127) >> 7;
  const int BH = p.B * p.H;
  // All query tiles of one (batch, head) pair are adjacent in the grid, heaviest first: the CTAs in
  // flight at any time stream the same few K/V tensors, which therefore stay in the L2 cache.
  // (With the pair as the fast index every resident CTA would stream a different pair from HBM.)
  const int bh = (int)(blockIdx.x / nmt);
  const int mt = nmt - 1 - (int)(blockIdx.x % nmt);
  const int b = bh / p.H, h = bh % p.H;
  const int len = p.varlen ? min(max(p.varlen[b], 0), L) : L;
  const int row0 = mt * 128;
  const bool tile_live = row0 < len;
  const int nkt = tile_live ? (causal ? min((len + 127) >> 7, mt + 1) : ((len + 127) >> 7)) : 0;
  const bool want_dbias = MODE == LAZY && p.dbias_acc != nullptr;
  volatile int* abort_flag = &sh.abort_flag;
  if (tid == 0) kernel_clock(status, 1, false);

  if (tid == 0) {
    mbar_init(&sh.res_full, 1);
    for (int s = 0; s < 3; ++s) {
      mbar_init(&sh.k_full[s], 1);
      mbar_init(&sh.k_empty[s], 1);      // committed by the last product that reads the K tile
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&sh.v_full[s], 1);
      mbar_init(&sh.v_empty[s], 1);      // ... the V tile
      mbar_init(&sh.t_full[s], 2);       // S and dP of a first-sweep tile, one commit each
      mbar_init(&sh.t_free[s], kBwdRowWarps);
      mbar_init(&sh.dp_full[s], 1);
      mbar_init(&sh.ds_full[s], kBwdRowWarps);
      mbar_init(&sh.dq_done[s], 1);
    }
    mbar_init(&sh.sweep_done, kBwdRowWarps);
    mbar_init(&sh.s_full, 1);
    mbar_init(&sh.s_free, kBwdRowWarps);
    mbar_init(&sh.acc_full, 1);
    sh.abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0) {
    const int n = build_tile_list(sh.tiles, nkt, p.block_mask == nullptr ? nullptr
                                  : p.block_mask + ((int64_t)bh * nmt + mt) * p.mask_words, lane);
    if (lane == 0) sh.nact = n;
  }
  if (warp == kBwdProducerWarp) tmem_alloc(&sh.tmem_base, 512);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = sh.tmem_base;
  const uint32_t tmem_acc = tmem + 384;
  const int nact = sh.nact;

  if (warp == kBwdProducerWarp) {
    if (lane == 0 && tile_live) {
      tma_prefetch_desc(&map_q); tma_prefetch_desc(&map_k); tma_prefetch_desc(&map_v); tma_prefetch_desc(&map_do);
      mbar_expect_tx(&sh.res_full, 2 * Cfg::kTileBytes);
      tma_load_tile<D>(sQ, &map_q, &sh.res_full, row0, h, b);
      tma_load_tile<D>(sdO, &map_do, &sh.res_full, row0, h, b);
      for (int g = 0; g < 2 * nact; ++g) {   // both sweeps
        const int s = g & 1, ks = k_slot(g), kt = sh.tiles[g < nact ? g : g - nact];
        // the K half of a slot is free after the S product (first sweep) or the dQ product (second
        // sweep), the V half after the dP product: each is refilled as soon as its own reader is done
        if (!mbar_wait(&sh.k_empty[ks], k_phase(g) ^ 1u, abort_flag, status, 40)) break;
        mbar_expect_tx(&sh.k_full[ks], Cfg::kTileBytes);
        tma_load_tile<D>(ring + ks * Cfg::kTileBytes, &map_k, &sh.k_full[ks], kt * 128, h / p.n_rep, b);   // (kv head)
        if (!mbar_wait(&sh.v_empty[s], ((g >> 1) & 1) ^ 1, abort_flag, status, 40)) break;
        mbar_expect_tx(&sh.v_full[s], Cfg::kTileBytes);
        tma_load_tile<D>(ring + (NK + s) * Cfg::kTileBytes, &map_v, &sh.v_full[s], kt * 128, h / p.n_rep, b);
      }
    }
    __syncwarp();
  } else if (warp >= kBwdProducerWarp + 1 && warp <= kBwdProducerWarp + 3) {
    if (lane == 0 && tile_live) {
      const int role = warp - (kBwdProducerWarp + 1);   // 0: S products, 1: dP products, 2: dQ products
      const uint32_t q_addr = smem_u32(sQ), do_addr = smem_u32(sdO), ring_addr = smem_u32(ring);
      // g counts tile pairs over both sweeps; ring stage and barrier phases follow g.  Every full /
      // empty barrier has one waiter, which sees each of its phases: K full -> the S thread, V full
      // -> the dP thread; the dQ thread needs no wait of its own for K (its dS operand exists only
      // after S of the same tile, i.e. after the K tile landed).
      auto k_addr = [&](int g) { return ring_addr + k_slot(g) * Cfg::kTileBytes; };
      auto v_addr = [&](int g) { return ring_addr + (NK + (g & 1)) * Cfg::kTileBytes; };
      bool ok = mbar_wait(&sh.res_full, 0, abort_flag, status, 41);
      // ---- first sweep: S and dP of tile g into slot g & 1 -----------------------------------
      if (role < 2) {
        for (int g = 0; g < nact; ++g) {
          const int j = g & 1;
          ok = ok && (role == 0 ? mbar_wait(&sh.k_full[k_slot(g)], k_phase(g), abort_flag, status, 42)
                                : mbar_wait(&sh.v_full[j], (g >> 1) & 1, abort_flag, status, 42));
          ok = ok && mbar_wait(&sh.t_free[j], ((g >> 1) & 1) ^ 1, abort_flag, status, 43);
          tc_fence_after_sync();
          if (ok) {
            if (role == 0) issue_nt<D, FMT>(tmem + 256 * j, q_addr, k_addr(g));
            else issue_nt<D, FMT>(tmem + 256 * j + 128, do_addr, v_addr(g));
          }
          umma_commit(&sh.t_full[j]);
          umma_commit(role == 0 ? &sh.k_empty[k_slot(g)] : &sh.v_empty[j]);
        }
      }
      // the second sweep lays tensor memory out differently: every first-sweep tile must be read
      ok = ok && mbar_wait(&sh.sweep_done, 0, abort_flag, status, 44);
      // ---- second sweep ---------------------------------------------------------------------------
      if (role == 0) {
        for (int t = 0; t < nact; ++t) {
          const int g = nact + t;
          ok = ok && mbar_wait(&sh.k_full[k_slot(g)], k_phase(g), abort_flag, status, 45);
          ok = ok && mbar_wait(&sh.s_free, (t & 1) ^ 1, abort_flag, status, 46);   // S of tile t-1 is in registers
          tc_fence_after_sync();
          if (ok) issue_nt<D, FMT>(tmem, q_addr, k_addr(g));
          umma_commit(&sh.s_full);
        }
      } else if (role == 1) {
        for (int t = 0; t < nact; ++t) {
          const int g = nact + t, bsel = t & 1;
          ok = ok && mbar_wait(&sh.v_full[g & 1], (g >> 1) & 1, abort_flag, status, 47);
          // dS of tile t-2 has been consumed before its buffer receives dP of tile t
          if (t >= 2) ok = ok && mbar_wait(&sh.dq_done[bsel], ((t - 2) >> 1) & 1, abort_flag, status, 48);
          tc_fence_after_sync();
          if (ok) issue_nt<D, FMT>(tmem + 128 + 128 * bsel, do_addr, v_addr(g));
          umma_commit(&sh.dp_full[bsel]);
          umma_commit(&sh.v_empty[g & 1]);
        }
      } else {
        for (int t = 0; t < nact; ++t) {   // dQ += dS(t) . K(t)
          const int g = nact + t, bsel = t & 1;
          ok = ok && mbar_wait(&sh.ds_full[bsel], (t >> 1) & 1, abort_flag, status, 50);
          tc_fence_after_sync();
          // keys beyond the end of the sequence: padding rows of K stay out of the reduction
          // (S of this tile has completed: dS exists), see zero_tail_rows
          int nks = 8;
          const int valid = len - (int)sh.tiles[t] * 128;
          if (ok && valid < 128) nks = zero_tail_rows(ring + k_slot(g) * Cfg::kTileBytes, valid, Cfg::kBoxes, 128);
          if (ok) issue_tn_quads<D, FMT>(tmem_acc, tmem + 128 + 128 * bsel, k_addr(g), t > 0, nks);
          umma_commit(&sh.dq_done[bsel]);
          umma_commit(&sh.k_empty[k_slot(g)]);
        }
        umma_commit(&sh.acc_full);
      }
      if (status) atomicAdd((unsigned long long*)(status + 4), (unsigned long long)(role < 2 ? 2 * nact : nact));
    }
    __syncwarp();
  } else {
    const int quad = warp >> 2;
    const int c0 = quad * 32;                 // first key column of this thread inside a tile
    const int row = (warp & 3) * 32 + lane;
    const int i = row0 + row;
    const bool live = i < len;
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    const int64_t bhl = (int64_t)bh * L;
    uint8_t* grow = (uint8_t*)p.dq.ptr + 2 * ((int64_t)b * p.dq.s[0] + (int64_t)h * p.dq.s[1] + (int64_t)i * p.dq.s[2]);
    if (tile_live) {
      const int jlim = live ? (causal ? min(i, len - 1) : len - 1) : -1;
      const int tile_jlim = (row0 + 127 < len) ? (causal ? row0 : len - 1) : -1;
      const float c1 = p.scale * (MODE == ENTMAX ? (p.alpha - 1.f) : kLog2e);
      const float e = MODE == ENTMAX ? 1.f / (p.alpha - 1.f) : 0.f;
      const float rstat = live ? (MODE == ENTMAX ? p.tau[bhl + i] : p.lse[bhl + i]) : 0.f;
      const float tau_row = MODE == LAZY ? p.tau_h[h] / (float)(i + 1) : 0.f;

      // ---- first sweep: the row scalars ---------------------------------------------------------
      float acc_a0 = 0.f, acc_a1 = 0.f, acc_b0 = 0.f, acc_b1 = 0.f;  // entmax: sum U dP, sum U; lazy: sum P M dP, sum M dP
      for (int g = 0; g < nact; ++g) {
        const int kt = sh.tiles[g], j = g & 1;
        const bool need_mask = kt * 128 + 127 > tile_jlim;
        const int climit = jlim - kt * 128 - c0;
        const bool in_window = MODE == LAZY && (row0 - kt * 128 - 127 < p.window);
        mbar_wait(&sh.t_full[j], (g >> 1) & 1, abort_flag, status, 52);
        __syncwarp();
        tc_fence_after_sync();
        const uint32_t t_s = tmem + lane_base + 256 * j + c0, t_dp = t_s + 128;
        // this thread's 32 columns of S and dP go to registers first, so that the slot is handed back
        // before any arithmetic and the products of tile g+2 can follow those of tile g+1 without a gap
        uint32_t r[32], gq[32];
        tmem_ld32(t_s, r);
        tmem_ld32(t_dp, gq);
        tmem_ld_wait_regs32(r);
        tmem_ld_wait_regs32(gq);
        tc_fence_before_sync();
        __syncwarp();
        float nrs = -rstat;
        if (lane == 0) {
          nrs = __uint_as_float(mbar_arrive_token(&sh.t_free[j])) - rstat;   // (token: see mbar_arrive_token)
          if (g == nact - 1) mbar_arrive(&sh.sweep_done);
        }
        if (MODE == ENTMAX && KIND == 0 && !need_mask) {
          // alpha = 1.5, no masked entry: U = max(x, 0) by one saturating fma; packed sums
          uint64_t sa = pack2(acc_a0, acc_a1), sb = pack2(acc_b0, acc_b1);
#pragma unroll
          for (int x = 0; x < 32; x += 2) {
            const float e0 = __saturatef(fmaf(__uint_as_float(r[x]), c1, nrs));
            const float e1 = __saturatef(fmaf(__uint_as_float(r[x + 1]), c1, nrs));
            const uint64_t ee = pack2(e0, e1);
            sa = fma2(ee, pack2(__uint_as_float(gq[x]), __uint_as_float(gq[x + 1])), sa);
            sb = add2(sb, ee);
          }
          unpack2(sa, acc_a0, acc_a1);
          unpack2(sb, acc_b0, acc_b1);
        } else if (MODE == LAZY && !need_mask && !in_window) {
          // interior tile (no masked entry, no bias): straight-line arithmetic on pairs (packed f32x2 operations
          // halve the issue slots of everything but the two exponentials and the two comparisons)
          uint64_t sa = pack2(acc_a0, acc_a1), sb = pack2(acc_b0, acc_b1);
          const uint64_t c2 = pack2(c1, c1), n2 = pack2(nrs, nrs), t2 = pack2(tau_row, tau_row);
#pragma unroll
          for (int x = 0; x < 32; x += 2) {
            float x0, x1, t0, t1;
            unpack2(fma2(pack2(__uint_as_float(r[x]), __uint_as_float(r[x + 1])), c2, n2), x0, x1);
            const uint64_t ww = pack2(fast_exp2(x0), fast_exp2(x1));
            unpack2(add2(ww, t2), t0, t1);
            // M dP: a product with 1 or 0 (every dP of an interior tile is finite)
            const uint64_t md = mul2(pack2(t0 > 0.f ? 1.f : 0.f, t1 > 0.f ? 1.f : 0.f),
                                     pack2(__uint_as_float(gq[x]), __uint_as_float(gq[x + 1])));
            sa = fma2(ww, md, sa);
            sb = add2(sb, md);
          }
          unpack2(sa, acc_a0, acc_a1);
          unpack2(sb, acc_b0, acc_b1);
        } else {
#pragma unroll
          for (int x = 0; x < 32; ++x) {
            float xs = __uint_as_float(r[x]) * c1;
            if (MODE == LAZY && in_window) {
              const int dist = i - (kt * 128 + c0 + x);
              if (dist >= 0 && dist < p.window) xs = fmaf(__ldg(p.bias + (int64_t)h * p.bias_stride + dist), kLog2e, xs);
            }
            if (MODE == ENTMAX) xs = fmaf(__uint_as_float(r[x]), c1, -rstat); else xs -= rstat;
            const bool valid = !need_mask || x <= climit;
            float pv, w;
            bool m;
            prob_terms<MODE, KIND>(xs, e, tau_row, valid, pv, w, m);
            // (a masked dP comes from padding rows of V or dO and may be anything: selected, never multiplied)
            const float dp = (MODE == LAZY || m) ? __uint_as_float(gq[x]) : 0.f;
            if (MODE == ENTMAX) {
              if (x & 1) { acc_a1 = fmaf(w, dp, acc_a1); acc_b1 += w; } else { acc_a0 = fmaf(w, dp, acc_a0); acc_b0 += w; }
            } else {
              const float md = m ? dp : 0.f;
              if (x & 1) { acc_a1 = fmaf(w, md, acc_a1); acc_b1 += md; } else { acc_a0 = fmaf(w, md, acc_a0); acc_b0 += md; }
            }
          }
        }
      }
      if (nact == 0 && lane == 0) mbar_arrive(&sh.sweep_done);
      // The four threads of a row meet in tensor memory: all own the same lane.  Columns 384..391
      // are free from the moment every row thread has read the last first-sweep tile (the first
      // barrier) until the first dQ product, which needs the delta computed here.
      named_bar_sync(1, kBwdRowThreads);
      tmem_st2(tmem_acc + lane_base + 2 * quad, __float_as_uint(acc_a0 + acc_a1), __float_as_uint(acc_b0 + acc_b1));
      tmem_st_wait();
      tc_fence_before_sync();
      named_bar_sync(1, kBwdRowThreads);
      tc_fence_after_sync();
      float delta = 0.f;
      {
        uint32_t all4[8];
        tmem_ld8_sync(tmem_acc + lane_base, all4);
        const float sa = (__uint_as_float(all4[0]) + __uint_as_float(all4[2])) + (__uint_as_float(all4[4]) + __uint_as_float(all4[6]));
        const float sb = (__uint_as_float(all4[1]) + __uint_as_float(all4[3])) + (__uint_as_float(all4[5]) + __uint_as_float(all4[7]));
        if (MODE == ENTMAX) {
          delta = (live && sb > 0.f) ? sa / sb : 0.f;
        } else {
          delta = live ? sa : 0.f;
          if (p.dtau_acc != nullptr && quad == 0) {     // dtau_h += sum_i r_i / (i+1)
            float contrib = live ? sb / (float)(i + 1) : 0.f;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) contrib += __shfl_xor_sync(0xffffffffu, contrib, o);
            if (lane == 0 && contrib != 0.f) atomicAdd(p.dtau_acc + h, to_fixed(contrib));
          }
        }
        if (i < L && quad == 0) p.delta[bhl + i] = delta;
      }

      // ---- second sweep: dS and dQ ------------------------------------------------------------------
      for (int t = 0; t < nact; ++t) {
        const int kt = sh.tiles[t], bsel = t & 1;
        const bool need_mask = kt * 128 + 127 > tile_jlim;
        const int climit = jlim - kt * 128 - c0;
        const bool in_window = MODE == LAZY && (row0 - kt * 128 - 127 < p.window);
        const uint32_t t_s = tmem + lane_base + c0, t_dp = tmem + lane_base + 128 + 128 * bsel + c0;
        // S has a single buffer, so this thread's columns go to registers as soon as they exist and the
        // buffer is handed back before dP is even waited for; the S product of the next tile then
        // overlaps the rest of this one.
        uint32_t r[32], gq[32], pk[16];
        mbar_wait(&sh.s_full, t & 1, abort_flag, status, 54);
        __syncwarp();
        tc_fence_after_sync();
        tmem_ld32(t_s, r);
        tmem_ld_wait_regs32(r);
        tc_fence_before_sync();
        __syncwarp();
        float nrs = -rstat;
        if (lane == 0) nrs = __uint_as_float(mbar_arrive_token(&sh.s_free)) - rstat;
        mbar_wait(&sh.dp_full[bsel], (t >> 1) & 1, abort_flag, status, 55);
        __syncwarp();
        tc_fence_after_sync();
        tmem_ld32_sync(t_dp, gq);
        if (MODE == ENTMAX && KIND == 0 && !need_mask) {
          const uint64_t nd = pack2(-delta, -delta);
#pragma unroll
          for (int x = 0; x < 32; x += 2) {
            const float e0 = __saturatef(fmaf(__uint_as_float(r[x]), c1, nrs));
            const float e1 = __saturatef(fmaf(__uint_as_float(r[x + 1]), c1, nrs));
            float d0, d1;
            unpack2(mul2(pack2(e0, e1), add2(pack2(__uint_as_float(gq[x]), __uint_as_float(gq[x + 1])), nd)), d0, d1);
            pk[x >> 1] = pack16<FMT>(d0, d1);
          }
        } else if (MODE == LAZY && !need_mask && !in_window) {
          // interior tile: no masked entry, no bias and hence no dbias contribution
          const uint64_t c2 = pack2(c1, c1), n2 = pack2(nrs, nrs), t2 = pack2(tau_row, tau_row), nd = pack2(-delta, -delta);
#pragma unroll
          for (int x = 0; x < 32; x += 2) {
            float x0, x1, t0, t1, d0, d1;
            unpack2(fma2(pack2(__uint_as_float(r[x]), __uint_as_float(r[x + 1])), c2, n2), x0, x1);
            const uint64_t ww = pack2(fast_exp2(x0), fast_exp2(x1));
            unpack2(add2(ww, t2), t0, t1);
            const uint64_t md = mul2(pack2(t0 > 0.f ? 1.f : 0.f, t1 > 0.f ? 1.f : 0.f),
                                     pack2(__uint_as_float(gq[x]), __uint_as_float(gq[x + 1])));
            unpack2(mul2(ww, add2(md, nd)), d0, d1);
            pk[x >> 1] = pack16<FMT>(d0, d1);
          }
        } else {
          const bool dbias_tile = MODE == LAZY && want_dbias && in_window;   // the same for the whole CTA
          float diag_a = 0.f, diag_b = 0.f;
#pragma unroll
          for (int x = 0; x < 32; x += 2) {
            float dsv[2];
#pragma unroll
            for (int y = 0; y < 2; ++y) {
              const int c = x + y;
              float xs = __uint_as_float(r[c]) * c1;
              if (MODE == LAZY && in_window) {
                const int dist = i - (kt * 128 + c0 + c);
                if (dist >= 0 && dist < p.window) xs = fmaf(__ldg(p.bias + (int64_t)h * p.bias_stride + dist), kLog2e, xs);
              }
              if (MODE == ENTMAX) xs = fmaf(__uint_as_float(r[c]), c1, -rstat); else xs -= rstat;
              const bool valid = !need_mask || c <= climit;
              float pv, w;
              bool m;
              prob_terms<MODE, KIND>(xs, e, tau_row, valid, pv, w, m);
              const float dp = __uint_as_float(gq[c]);
              // masked entries: exactly zero, whatever dP holds there (padding may be NaN)
              const float ds = MODE == ENTMAX ? (m ? w * (dp - delta) : 0.f) : (valid ? w * ((m ? dp : 0.f) - delta) : 0.f);
              dsv[y] = ds;
              if (MODE == LAZY && dbias_tile) {
                // dbias: sums of dS along the diagonals i - j.  The lanes of a warp are 32 consecutive rows, so
                // for column c the lanes hold 32 consecutive distances; rotating the column by c lanes brings
                // the entries of one diagonal to one lane: lane l collects distance base + l from the lanes that
                // did not wrap around and base + l - 32 from those that did (fixed order: reproducible sums),
                // and the warp ends the tile with 64 additions to the accumulators in global memory.
                const int dist = i - (kt * 128 + c0 + c);
                const float dm = dist < p.window ? ds : 0.f;   // (ds = 0 wherever dist < 0: causal)
                const float got = __shfl_sync(0xffffffffu, dm, (lane + c) & 31);
                if (lane + c < 32) diag_a += got; else diag_b += got;
              }
            }
            pk[x >> 1] = pack16<FMT>(dsv[0], dsv[1]);
          }
          if (MODE == LAZY && dbias_tile) {
            const int base = row0 + (warp & 3) * 32 - kt * 128 - c0;   // distance of (lane 0, column 0)
#pragma unroll
            for (int part = 0; part < 2; ++part) {
              const float sum = part == 0 ? diag_a : diag_b;
              const int dist = base + lane - 32 * part;
              if (sum != 0.f && dist >= 0 && dist < p.window)
                atomicAdd(p.dbias_acc + (int64_t)h * p.dbias_acc_stride + dist, to_fixed(sum));
            }
          }
        }
        tmem_st16(t_dp, pk);
        tmem_st_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&sh.ds_full[bsel]);
      }
      mbar_wait(&sh.acc_full, 0, abort_flag, status, 56);   // (committed even when no tile was visited)
      __syncwarp();
      tc_fence_after_sync();
      // each of the four threads of a row stores a quarter of the dQ columns
      {
        uint32_t r[32];
        if (D == 128) tmem_ld32_sync(tmem_acc + lane_base + quad * 32, r);
        else { tmem_ld16(tmem_acc + lane_base + quad * 16, r); tmem_ld_wait_regs16(r); }
        if (i < L) {
#pragma unroll
          for (int x = 0; x < D / 4; x += 8) {
            uint4 w;
            w.x = (live && nact > 0) ? pack16<FMT>(__uint_as_float(r[x + 0]) * p.scale, __uint_as_float(r[x + 1]) * p.scale) : 0u;
            w.y = (live && nact > 0) ? pack16<FMT>(__uint_as_float(r[x + 2]) * p.scale, __uint_as_float(r[x + 3]) * p.scale) : 0u;
            w.z = (live && nact > 0) ? pack16<FMT>(__uint_as_float(r[x + 4]) * p.scale, __uint_as_float(r[x + 5]) * p.scale) : 0u;
            w.w = (live && nact > 0) ? pack16<FMT>(__uint_as_float(r[x + 6]) * p.scale, __uint_as_float(r[x + 7]) * p.scale) : 0u;
            *(uint4*)(grow + (quad * (D / 4) + x) * 2) = w;
          }
        }
      }
    } else if (i < L) {
#pragma unroll
      for (int x = 0; x < D / 4; x += 8) *(uint4*)(grow + (quad * (D / 4) + x) * 2) = make_uint4(0u, 0u, 0u, 0u);
    }
    tc_fence_before_sync();
  }

  __syncthreads();
  if (*abort_flag) {
    for (int w = 0; w < 2000; ++w) __nanosleep(1000);
  }
  if (tid == 0) kernel_clock(status, 1, true);
  if (warp == kBwdProducerWarp) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, 512);
  }
}

}  // namespace tc
}  // namespace fla
