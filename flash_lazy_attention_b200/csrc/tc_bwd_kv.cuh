// Tensor-core dK / dV kernel of alpha-entmax attention and Lazy Attention.
//
// One CTA per 128-key tile of one (batch, kv head); K and V stay in shared memory, the (Q, dO) tiles of
// 128 query rows of every query head that shares this kv head (one without grouped-query attention)
// stream through a two-stage ring and accumulate into the same dK and dV.  Scores are produced transposed (S^T = K.Q^T, dP^T = V.dO^T, 128 keys x
// 128 queries, one N = 128 product each) so that a thread owns a key row; per-query statistics (tau or
// lse, delta, tau_h/(i+1)) are staged in shared memory.
//
//   warps 0-15 row threads, four per key row, 32 of the 128 query columns each.  Two phases per tile:
//              S^T -> P^T (16-bit A operand, written over the first half of the columns the thread read;
//              the factor U stays in registers), then dP^T -> dS^T the same way;
//   warp 16    TMA producer;
//   warp 17    issues the score products S^T and dP^T;
//   warp 18    issues the accumulating products dV += P^T.dO and dK += dS^T.Q.
//
// Tensor-memory columns: S^T [0,128), dP^T [128,256), dK [256,256+D), dV [384,384+D): every column is in
// use and nothing is double-buffered.  The tensor pipe stays busy because the work of a tile comes in
// four products that free and fill the two score buffers alternately:
//     S^T(t) | dP^T(t) | dV(t) | S^T(t+1) , dK(t) | dP^T(t+1) | dV(t+1) | ...
// P^T(t) is formed while dP^T(t) runs, dS^T(t) while dV(t) runs; S^T(t+1) may start when dV(t) has read
// P^T(t), dP^T(t+1) when dK(t) has read dS^T(t).  (An earlier version ping-ponged two 64-query sub-tiles
// with N = 64 score products, which read the K and V operands twice per 128 queries.)
//
// Replaces lazy_attention_triton.py:398-497 and the dK/dV half of the adasplash backward (source
// absent from the reference checkout).  Reads the delta that dq_kernel stored.
#pragma once

#include "common.cuh"
#include "tc_bwd.cuh"
#include "tc_fwd.cuh"
#include "tc_prims.cuh"

namespace fla {
namespace tc {

constexpr int kKvThreads = 608;   // 16 row warps, the copy producer, two product issuers
constexpr int kKvRowThreads = 512;
constexpr int kKvRowWarps = 16;
constexpr int kKvProducerWarp = 16;
constexpr int kKvMmaWarp = 17;
constexpr int kKvStages = 2;
constexpr int kKvMaxTiles = 2048;   // (query head of the group, query tile) items per CTA

struct KvShared {
  uint64_t res_full, ring_full[kKvStages], ring_empty[kKvStages];
  uint64_t s_full, dp_full, p_full, ds_full, dv_done, dk_done, acc_full;
  uint32_t tmem_base;
  int abort_flag;
  float stat[2][3][128];     // double buffer, statistic, query column
  int nact;                  // number of (query head, query tile) items this CTA visits
  uint16_t tiles[kKvMaxTiles];    // query tile (128-row units) in the low 9 bits, head of the group above
};

template <int MODE, int D, int FMT, int KIND>
__global__ void __launch_bounds__(kKvThreads, 1)
dkdv_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
            const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do,
            const AttnParams p, int* status) {
  using Cfg = TileCfg<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align_1024(smem_raw);
  uint8_t* sK = smem;
  uint8_t* sV = smem + Cfg::kTileBytes;
  uint8_t* ring = smem + 2 * Cfg::kTileBytes;      // stage s: Q tile, then dO tile
  __shared__ KvShared sh;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool causal = (MODE == LAZY) ? true : (p.causal != 0);
  const int L = p.L;
  // all key tiles of one (batch, head) pair are adjacent in the grid, so that the CTAs in flight
  // stream the same Q/dO tensors out of the L2 cache; key tile 0 sees every query tile under the
  // causal mask: heaviest first
  const int nkt_grid = (L + 127) >> 7;
  const int bhk = (int)(blockIdx.x / nkt_grid);
  const int nt = (int)(blockIdx.x % nkt_grid);
  const int b = bhk / p.Hkv, hk = bhk % p.Hkv;     // kv head; its query heads are hk * n_rep + rep
  const int len = p.varlen ? min(max(p.varlen[b], 0), L) : L;
  const int col0 = nt * 128;
  const bool tile_live = col0 < len;
  const int qt_begin = causal ? nt : 0;            // first 128-row query tile
  const int qt_end = (len + 127) >> 7;
  const int nq_all = tile_live ? qt_end - qt_begin : 0;
  volatile int* abort_flag = &sh.abort_flag;
  if (tid == 0) kernel_clock(status, 2, false);

  if (tid == 0) {
    mbar_init(&sh.res_full, 1);
    for (int s = 0; s < kKvStages; ++s) { mbar_init(&sh.ring_full[s], 1); mbar_init(&sh.ring_empty[s], 1); }
    mbar_init(&sh.s_full, 1);
    mbar_init(&sh.dp_full, 1);
    mbar_init(&sh.p_full, kKvRowWarps);     // one arrival per row warp
    mbar_init(&sh.ds_full, kKvRowWarps);
    mbar_init(&sh.dv_done, 1);
    mbar_init(&sh.dk_done, 1);
    mbar_init(&sh.acc_full, 1);
    sh.abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0) {
    // items to visit: every query tile of every query head of the group, or those with a non-zero
    // probability in one of the two 64-key halves of this key tile according to the forward's block mask
    int n = 0;
    const int nmt = (L + 127) >> 7;
    for (int rep = 0; rep < p.n_rep; ++rep) {
      const int64_t bh = (int64_t)b * p.H + hk * p.n_rep + rep;
      for (int base = 0; base < nq_all; base += 32) {
        const int qt = qt_begin + base + lane;
        bool on = base + lane < nq_all;
        if (on && p.block_mask != nullptr) {
          const uint32_t w = p.block_mask[(bh * nmt + qt) * p.mask_words + ((2 * nt) >> 5)];
          on = ((w >> ((2 * nt) & 31)) & 3u) != 0u;
        }
        const uint32_t votes = __ballot_sync(0xffffffffu, on);
        if (on) sh.tiles[n + __popc(votes & ((1u << lane) - 1u))] = (uint16_t)((rep << 9) | qt);
        n += __popc(votes);
      }
    }
    if (lane == 0) sh.nact = n;
  }
  if (warp == kKvProducerWarp) tmem_alloc(&sh.tmem_base, 512);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = sh.tmem_base;
  const uint32_t tmem_dp = tmem + 128, tmem_dk = tmem + 256, tmem_dv = tmem + 384;
  const int nq = sh.nact;

  if (warp == kKvProducerWarp) {
    if (lane == 0 && tile_live) {
      tma_prefetch_desc(&map_q); tma_prefetch_desc(&map_k); tma_prefetch_desc(&map_v); tma_prefetch_desc(&map_do);
      mbar_expect_tx(&sh.res_full, 2 * Cfg::kTileBytes);
      tma_load_tile<D>(sK, &map_k, &sh.res_full, col0, hk, b);
      tma_load_tile<D>(sV, &map_v, &sh.res_full, col0, hk, b);
      for (int n = 0; n < nq; ++n) {
        const int s = n % kKvStages, q0 = (int)(sh.tiles[n] & 511u) * 128, h = hk * p.n_rep + (int)(sh.tiles[n] >> 9);
        uint8_t* dst = ring + s * 2 * Cfg::kTileBytes;
        if (!mbar_wait(&sh.ring_empty[s], ((n / kKvStages) & 1) ^ 1, abort_flag, status, 60)) break;
        mbar_expect_tx(&sh.ring_full[s], 2 * Cfg::kTileBytes);
        tma_load_tile<D>(dst, &map_q, &sh.ring_full[s], q0, h, b);
        tma_load_tile<D>(dst + Cfg::kTileBytes, &map_do, &sh.ring_full[s], q0, h, b);
      }
    }
    __syncwarp();
  } else if (warp == kKvMmaWarp || warp == kKvMmaWarp + 1) {
    // Two issuing threads: one for the score products S^T and dP^T, one for the accumulating
    // products dV and dK.  Each barrier below has a single waiting issuer, which sees every one of
    // its phases (all of them complete once per tile).
    if (lane == 0 && tile_live) {
      const uint32_t k_addr = smem_u32(sK), v_addr = smem_u32(sV), ring_addr = smem_u32(ring);
      bool ok = mbar_wait(&sh.res_full, 0, abort_flag, status, 61);
      if (warp == kKvMmaWarp) {
        for (int n = 0; n < nq; ++n) {
          const int s = n % kKvStages;
          const uint32_t q_addr = ring_addr + s * 2 * Cfg::kTileBytes, do_addr = q_addr + Cfg::kTileBytes;
          ok = ok && mbar_wait(&sh.ring_full[s], (n / kKvStages) & 1, abort_flag, status, 62);
          // S^T(n) over P^T(n-1): free once dV(n-1) has read it
          if (n > 0) ok = ok && mbar_wait(&sh.dv_done, (n - 1) & 1, abort_flag, status, 63);
          tc_fence_after_sync();
          if (ok) issue_nt<D, FMT>(tmem, k_addr, q_addr);                 // S^T  = K . Q^T
          umma_commit(&sh.s_full);
          // dP^T(n) over dS^T(n-1): free once dK(n-1) has read it
          if (n > 0) ok = ok && mbar_wait(&sh.dk_done, (n - 1) & 1, abort_flag, status, 68);
          tc_fence_after_sync();
          if (ok) issue_nt<D, FMT>(tmem_dp, v_addr, do_addr);             // dP^T = V . dO^T
          umma_commit(&sh.dp_full);
        }
        if (status) atomicAdd((unsigned long long*)(status + 4), (unsigned long long)(2 * nq));
      } else {
        for (int n = 0; n < nq; ++n) {
          const int s = n % kKvStages;
          const uint32_t q_addr = ring_addr + s * 2 * Cfg::kTileBytes, do_addr = q_addr + Cfg::kTileBytes;
          ok = ok && mbar_wait(&sh.p_full, n & 1, abort_flag, status, 64);
          tc_fence_after_sync();
          // query rows beyond the end of the sequence: padding rows of Q and dO stay out of the
          // reductions (the score products of this tile have completed), see zero_tail_rows
          int nks = 8;
          const int valid = len - (int)(sh.tiles[n] & 511u) * 128;
          if (ok && valid < 128) {
            uint8_t* stage = ring + s * 2 * Cfg::kTileBytes;
            zero_tail_rows(stage, valid, Cfg::kBoxes, 128);
            nks = zero_tail_rows(stage + Cfg::kTileBytes, valid, Cfg::kBoxes, 128);
          }
          if (ok) issue_tn_quads<D, FMT>(tmem_dv, tmem, do_addr, n > 0, nks);        // dV += P^T . dO
          umma_commit(&sh.dv_done);
          ok = ok && mbar_wait(&sh.ds_full, n & 1, abort_flag, status, 65);
          tc_fence_after_sync();
          if (ok) issue_tn_quads<D, FMT>(tmem_dk, tmem_dp, q_addr, n > 0, nks);      // dK += dS^T . Q
          umma_commit(&sh.dk_done);
          umma_commit(&sh.ring_empty[s]);
        }
        umma_commit(&sh.acc_full);
        if (status) atomicAdd((unsigned long long*)(status + 4), (unsigned long long)(2 * nq));
      }
    }
    __syncwarp();
  } else {
    // Sixteen row warps: four threads per key row, thread `quad` taking query columns [32 quad, +32).
    const int quad = warp >> 2;
    const int row = (warp & 3) * 32 + lane;
    const int j = col0 + row;
    const bool live = j < len;
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    // my 32 score columns; P^T / dS^T (16-bit pairs) go to the first 16 of them
    const uint32_t t_s = tmem + lane_base + quad * 32, t_dp = t_s + 128;
    if (tile_live) {
      const float c1 = p.scale * (MODE == ENTMAX ? (p.alpha - 1.f) : kLog2e);
      const float e = MODE == ENTMAX ? 1.f / (p.alpha - 1.f) : 0.f;
      const float* gstat = MODE == ENTMAX ? p.tau : p.lse;
      // The statistics of a tile's 128 query rows are fetched one tile ahead (threads 0-127, one row
      // each): the loads from global memory are in flight while the previous tile is worked on.
      // entmax keeps the negated values: they are the addends of  x = s*c1 - tau  and  dP - delta.
      const float sgn = -1.f;   // the row statistic and delta are staged negated: both only ever get subtracted
      float nx_stat = 0.f, nx_delta = 0.f;
      auto fetch_stats = [&](int n) {
        if (tid < 128 && n < nq) {
          const int qi = (int)(sh.tiles[n] & 511u) * 128 + tid;
          const int64_t bhl = ((int64_t)b * p.H + hk * p.n_rep + (int)(sh.tiles[n] >> 9)) * L;
          const bool ql = qi < len;
          nx_stat = ql ? sgn * gstat[bhl + qi] : 0.f;
          nx_delta = ql ? sgn * p.delta[bhl + qi] : 0.f;
        }
      };
      fetch_stats(0);
      for (int n = 0; n < nq; ++n) {
        const int q0 = (int)(sh.tiles[n] & 511u) * 128;
        const int h = hk * p.n_rep + (int)(sh.tiles[n] >> 9);    // query head of this item
        float (*st)[128] = sh.stat[n & 1];
        if (tid < 128) {
          st[0][tid] = nx_stat;
          st[1][tid] = nx_delta;
          st[2][tid] = MODE == LAZY ? p.tau_h[h] / (float)(q0 + tid + 1) : 0.f;
        }
        fetch_stats(n + 1);
        named_bar_sync(1, kKvRowThreads);
        const int cb = quad * 32;                    // first query column of this thread
        // query column c (row q0 + c) may use key j iff cmin <= c <= cmax
        const int cmax = live ? min(127, len - 1 - q0) : -1;
        const int cmin = causal ? j - q0 : 0;
        const bool need_mask = (causal && q0 < col0 + 128) || (q0 + 127 >= len) || (col0 + 127 >= len);
        const bool in_window = MODE == LAZY && (q0 - col0 - 127 < p.window);
        const float* s0 = st[0] + cb;
        const float* s1 = st[1] + cb;
        const float* s2 = st[2] + cb;
        const bool fast = (MODE == ENTMAX && KIND == 0 && !need_mask) || (MODE == LAZY && !need_mask && !in_window);
        float w[32];            // U (entmax) or the softmax probability (lazy): the factor of dS
        uint32_t vmask = 0xffffffffu, mmask = 0xffffffffu;   // general path: valid entries / support
        uint32_t r[32], pk[16];
        // ---- phase 1: S^T -> P^T ---------------------------------------------------------------
        mbar_wait(&sh.s_full, n & 1, abort_flag, status, 66);
        __syncwarp();
        tc_fence_after_sync();
        tmem_ld32_sync(t_s, r);
        if (fast && MODE == ENTMAX) {
          // alpha = 1.5, no masked entry: U = max(x, 0) by one saturating fma (x <= 1 everywhere), P = U^2
#pragma unroll
          for (int x = 0; x < 32; x += 2) {
            w[x] = __saturatef(fmaf(__uint_as_float(r[x]), c1, s0[x]));
            w[x + 1] = __saturatef(fmaf(__uint_as_float(r[x + 1]), c1, s0[x + 1]));
            pk[x >> 1] = pack16<FMT>(w[x] * w[x], w[x + 1] * w[x + 1]);
          }
        } else if (fast) {
          // lazy, interior tile: no masked entry and no bias, straight-line arithmetic on pairs.  w keeps the
          // softmax probability with the ReLU mask in its sign (negative: A = 0 there), which is all phase 2 needs.
          const uint64_t c2 = pack2(c1, c1);
#pragma unroll
          for (int x = 0; x < 32; x += 2) {
            float x0, x1, t0, t1;
            unpack2(fma2(pack2(__uint_as_float(r[x]), __uint_as_float(r[x + 1])), c2,
                         *reinterpret_cast<const uint64_t*>(s0 + x)), x0, x1);
            const float w0 = fast_exp2(x0), w1 = fast_exp2(x1);
            unpack2(add2(pack2(w0, w1), *reinterpret_cast<const uint64_t*>(s2 + x)), t0, t1);
            w[x] = t0 > 0.f ? w0 : -w0;
            w[x + 1] = t1 > 0.f ? w1 : -w1;
            pk[x >> 1] = pack16<FMT>(fmaxf(t0, 0.f), fmaxf(t1, 0.f));
          }
        } else {
          vmask = 0u;
          mmask = 0u;
#pragma unroll
          for (int x = 0; x < 32; x += 2) {
            float pvv[2];
#pragma unroll
            for (int y = 0; y < 2; ++y) {
              const int c = cb + x + y;
              float xs;
              if (MODE == ENTMAX) {
                xs = fmaf(__uint_as_float(r[x + y]), c1, s0[x + y]);
              } else {
                xs = __uint_as_float(r[x + y]) * c1;
                if (in_window) {
                  const int dist = q0 + c - j;
                  if (dist >= 0 && dist < p.window) xs = fmaf(__ldg(p.bias + (int64_t)h * p.bias_stride + dist), kLog2e, xs);
                }
                xs += s0[x + y];
              }
              const bool valid = !need_mask || (c >= cmin && c <= cmax);
              float pv, wv;
              bool m;
              prob_terms<MODE, KIND>(xs, e, s2[x + y], valid, pv, wv, m);
              pvv[y] = pv;
              w[x + y] = wv;
              vmask |= (valid ? 1u : 0u) << (x + y);
              mmask |= (m ? 1u : 0u) << (x + y);
            }
            pk[x >> 1] = pack16<FMT>(pvv[0], pvv[1]);
          }
        }
        tmem_st16(t_s, pk);
        tmem_st_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&sh.p_full);
        // ---- phase 2: dP^T -> dS^T ---------------------------------------------------------------
        mbar_wait(&sh.dp_full, n & 1, abort_flag, status, 69);
        __syncwarp();
        tc_fence_after_sync();
        tmem_ld32_sync(t_dp, r);
        if (fast && MODE == ENTMAX) {
#pragma unroll
          for (int x = 0; x < 32; x += 2) {
            float d0, d1;
            unpack2(mul2(pack2(w[x], w[x + 1]), add2(pack2(__uint_as_float(r[x]), __uint_as_float(r[x + 1])),
                                                      *reinterpret_cast<const uint64_t*>(s1 + x))), d0, d1);
            pk[x >> 1] = pack16<FMT>(d0, d1);
          }
        } else if (fast) {
          // lazy, interior tile: dS = P (M dP - delta), M in the sign of w (every dP of an interior tile is finite)
#pragma unroll
          for (int x = 0; x < 32; x += 2) {
            float e0, e1;
            const uint64_t md = mul2(pack2(w[x] > 0.f ? 1.f : 0.f, w[x + 1] > 0.f ? 1.f : 0.f),
                                     pack2(__uint_as_float(r[x]), __uint_as_float(r[x + 1])));
            unpack2(add2(md, *reinterpret_cast<const uint64_t*>(s1 + x)), e0, e1);
            pk[x >> 1] = pack16<FMT>(fabsf(w[x]) * e0, fabsf(w[x + 1]) * e1);
          }
        } else {
#pragma unroll
          for (int x = 0; x < 32; x += 2) {
            float dsv[2];
#pragma unroll
            for (int y = 0; y < 2; ++y) {
              const float dp = __uint_as_float(r[x + y]);
              const bool valid = (vmask >> (x + y)) & 1u, m = (mmask >> (x + y)) & 1u;
              // masked entries: exactly zero, whatever dP holds there (padding may be NaN)
              dsv[y] = MODE == ENTMAX ? (m ? w[x + y] * (dp + s1[x + y]) : 0.f)
                                      : (valid ? w[x + y] * ((m ? dp : 0.f) + s1[x + y]) : 0.f);
            }
            pk[x >> 1] = pack16<FMT>(dsv[0], dsv[1]);
          }
        }
        tmem_st16(t_dp, pk);
        tmem_st_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&sh.ds_full);
      }
      mbar_wait(&sh.acc_full, 0, abort_flag, status, 67);   // (committed even when no tile was visited)
      __syncwarp();
      tc_fence_after_sync();
      // quads 0, 1 store dK, quads 2, 3 store dV; each takes half of the columns
      const int grp = quad >> 1, half = quad & 1;
      uint8_t* grow = (uint8_t*)(grp == 0 ? p.dk.ptr : p.dv.ptr) +
                      2 * ((int64_t)b * (grp == 0 ? p.dk.s[0] : p.dv.s[0]) + (int64_t)hk * (grp == 0 ? p.dk.s[1] : p.dv.s[1]) +
                           (int64_t)j * (grp == 0 ? p.dk.s[2] : p.dv.s[2]));
      const float mul = grp == 0 ? p.scale : 1.f;
#pragma unroll
      for (int cc = 0; cc < D / 64; ++cc) {
        const int ch = half * (D / 64) + cc;
        uint32_t o[32];
        tmem_ld32_sync((grp == 0 ? tmem_dk : tmem_dv) + lane_base + ch * 32, o);
        if (j < L) {
#pragma unroll
          for (int x = 0; x < 32; x += 8) {
            uint4 wv;
            wv.x = (live && nq > 0) ? pack16<FMT>(__uint_as_float(o[x + 0]) * mul, __uint_as_float(o[x + 1]) * mul) : 0u;
            wv.y = (live && nq > 0) ? pack16<FMT>(__uint_as_float(o[x + 2]) * mul, __uint_as_float(o[x + 3]) * mul) : 0u;
            wv.z = (live && nq > 0) ? pack16<FMT>(__uint_as_float(o[x + 4]) * mul, __uint_as_float(o[x + 5]) * mul) : 0u;
            wv.w = (live && nq > 0) ? pack16<FMT>(__uint_as_float(o[x + 6]) * mul, __uint_as_float(o[x + 7]) * mul) : 0u;
            *(uint4*)(grow + (ch * 32 + x) * 2) = wv;
          }
        }
      }
    } else if (j < L) {
      const int grp = quad >> 1, half = quad & 1;
      uint8_t* grow = (uint8_t*)(grp == 0 ? p.dk.ptr : p.dv.ptr) +
                      2 * ((int64_t)b * (grp == 0 ? p.dk.s[0] : p.dv.s[0]) + (int64_t)hk * (grp == 0 ? p.dk.s[1] : p.dv.s[1]) +
                           (int64_t)j * (grp == 0 ? p.dk.s[2] : p.dv.s[2]));
#pragma unroll
      for (int x = 0; x < D / 2; x += 8) *(uint4*)(grow + (half * (D / 2) + x) * 2) = make_uint4(0u, 0u, 0u, 0u);
    }
    tc_fence_before_sync();
  }

  __syncthreads();
  if (*abort_flag) {
    for (int w = 0; w < 2000; ++w) __nanosleep(1000);
  }
  if (tid == 0) kernel_clock(status, 2, true);
  if (warp == kKvProducerWarp) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, 512);
  }
}

}  // namespace tc
}  // namespace fla
