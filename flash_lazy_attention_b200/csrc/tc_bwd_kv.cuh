// Tensor-core dK / dV kernel of alpha-entmax attention and Lazy Attention.
//
// One CTA per 128-key tile; K and V stay in shared memory, (Q, dO) sub-tiles of 64 query rows
// stream through a four-stage ring.  Scores are produced transposed (S^T = K.Q^T, dP^T = V.dO^T,
// 128 keys x 64 queries) so that a thread owns a key row; per-query statistics (tau or lse,
// delta, tau_h/(i+1)) are staged in shared memory.
//
//   warps 0-15 two groups; group g owns the score buffers g and handles every second sub-tile, two
//              threads per key row (32 of the 64 query columns each): P^T overwrites S^T, dS^T
//              overwrites dP^T (16-bit A operands), each thread inside the columns it read;
//   warp 16    TMA producer;
//   warp 17    issues the score products S^T and dP^T;
//   warp 18    issues the accumulating products dV += P^T.dO and dK += dS^T.Q; one group's
//              arithmetic overlaps the other group's tensor work.
//
// Tensor-memory columns: S^T buffers [0,64) and [64,128), dP^T buffers [128,192) and [192,256),
// dK [256,256+D), dV [384,384+D).
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
constexpr int kKvGroupThreads = 256;
constexpr int kKvGroupWarps = 8;
constexpr int kKvProducerWarp = 16;
constexpr int kKvMmaWarp = 17;
constexpr int kKvStages = 4;

struct KvShared {
  uint64_t res_full, ring_full[kKvStages], ring_empty[kKvStages];
  uint64_t sdp_full[2], p_full[2], ds_full[2], kd_done[2], acc_full;
  uint32_t tmem_base;
  int abort_flag;
  float stat[2][2][3][64];   // group, double buffer, statistic, query column
  int nact;                  // number of query sub-tiles this CTA visits
  uint16_t subs[2048];       // their indices (64-row units), ascending
};

// D[128 x N] = A[128 x D] . B[N x D]^T, K-major tiles; a_box / b_box: bytes of one 64-column box.
template <int D, int FMT, int N>
__device__ __forceinline__ void issue_nt_n(uint32_t d_tmem, uint32_t a_addr, uint32_t a_box, uint32_t b_addr,
                                           uint32_t b_box) {
  constexpr uint32_t idesc = make_idesc(128, N, FMT, 0, 0);
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks)
    umma_ss(d_tmem, desc_kmajor(a_addr + (ks >> 2) * a_box + (ks & 3) * 32),
            desc_kmajor(b_addr + (ks >> 2) * b_box + (ks & 3) * 32), idesc, ks > 0);
}

// D[128 x D] (+)= A[128 x KR] . B[KR x D]: A in tensor memory (16-bit pairs), B a [KR rows x D]
// tile whose rows are the reduction dimension; b_box = bytes of one 64-column box (KR * 128).
// The 16-bit A operand comes in two pieces: reduction rows 0..KR/2-1 at a_tmem, the rest 32 columns
// further on (each of the two threads of a key row writes its half inside the columns it read).
// `nks`: 16-row steps to issue (fewer for the sub-tile that reaches into a sequence's padding).
template <int D, int FMT, int KR>
__device__ __forceinline__ void issue_tn_k(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_addr, uint32_t b_box,
                                           bool accumulate, int nks = KR / 16) {
  constexpr uint32_t idesc = make_idesc(128, D, FMT, 0, 1);
  constexpr int kSteps = KR / 16;
#pragma unroll
  for (int ks = 0; ks < kSteps; ++ks)
    if (ks < nks)
      umma_ts(d_tmem, a_tmem + (ks < kSteps / 2 ? ks * 8 : 32 + (ks - kSteps / 2) * 8), desc_mnmajor(b_addr + ks * 2048, b_box),
              idesc, (accumulate || ks > 0) ? 1u : 0u);
}

template <int MODE, int D, int FMT, int KIND>
__global__ void __launch_bounds__(kKvThreads, 1)
dkdv_kernel(const __grid_constant__ CUtensorMap map_q64, const __grid_constant__ CUtensorMap map_k,
            const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do64,
            const AttnParams p, int* status) {
  using Cfg = TileCfg<D>;
  constexpr int kSubBytes = Cfg::kTileBytes / 2;   // a 64 x D sub-tile
  constexpr int kSubBox = 64 * 128;                // one 64-column box of it
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align_1024(smem_raw);
  uint8_t* sK = smem;
  uint8_t* sV = smem + Cfg::kTileBytes;
  uint8_t* ring = smem + 2 * Cfg::kTileBytes;      // stage s: Q sub-tile, then dO sub-tile
  __shared__ KvShared sh;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool causal = (MODE == LAZY) ? true : (p.causal != 0);
  const int L = p.L;
  const int BH = p.B * p.H;
  // key tile 0 sees every query tile under the causal mask: heaviest first
  // all key tiles of one (batch, head) pair are adjacent in the grid, so that the CTAs in flight
  // stream the same Q/dO tensors out of the L2 cache
  const int nkt_grid = (L + 127) >> 7;
  const int bh = (int)(blockIdx.x / nkt_grid);
  const int nt = (int)(blockIdx.x % nkt_grid);
  const int b = bh / p.H, h = bh % p.H;
  const int len = p.varlen ? min(max(p.varlen[b], 0), L) : L;
  const int col0 = nt * 128;
  const bool tile_live = col0 < len;
  const int n_begin = causal ? 2 * nt : 0;         // first 64-row query sub-tile
  const int n_end = (len + 63) >> 6;
  const int nq_all = tile_live ? n_end - n_begin : 0;
  volatile int* abort_flag = &sh.abort_flag;
  if (tid == 0) kernel_clock(status, 2, false);

  if (tid == 0) {
    mbar_init(&sh.res_full, 1);
    for (int s = 0; s < kKvStages; ++s) { mbar_init(&sh.ring_full[s], 1); mbar_init(&sh.ring_empty[s], 1); }
    for (int g = 0; g < 2; ++g) {
      mbar_init(&sh.sdp_full[g], 1);
      mbar_init(&sh.p_full[g], kKvGroupWarps);    // one arrival per warp of the group
      mbar_init(&sh.ds_full[g], kKvGroupWarps);
      mbar_init(&sh.kd_done[g], 1);
    }
    mbar_init(&sh.acc_full, 1);
    sh.abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0) {
    // sub-tiles to visit: all, or those whose 128-row query block has a non-zero probability in
    // one of the two 64-key halves of this key tile according to the forward's block mask
    int n = 0;
    const int nmt = (L + 127) >> 7;
    for (int base = 0; base < nq_all; base += 32) {
      const int sub = n_begin + base + lane;
      bool on = base + lane < nq_all;
      if (on && p.block_mask != nullptr) {
        const uint32_t w = p.block_mask[((int64_t)bh * nmt + (sub >> 1)) * p.mask_words + ((2 * nt) >> 5)];
        on = ((w >> ((2 * nt) & 31)) & 3u) != 0u;
      }
      const uint32_t votes = __ballot_sync(0xffffffffu, on);
      if (on) sh.subs[n + __popc(votes & ((1u << lane) - 1u))] = (uint16_t)sub;
      n += __popc(votes);
    }
    if (lane == 0) sh.nact = n;
  }
  if (warp == kKvProducerWarp) tmem_alloc(&sh.tmem_base, 512);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = sh.tmem_base;
  const uint32_t tmem_dk = tmem + 256, tmem_dv = tmem + 384;
  const int nq = sh.nact;

  if (warp == kKvProducerWarp) {
    if (lane == 0 && tile_live) {
      tma_prefetch_desc(&map_q64); tma_prefetch_desc(&map_k); tma_prefetch_desc(&map_v); tma_prefetch_desc(&map_do64);
      mbar_expect_tx(&sh.res_full, 2 * Cfg::kTileBytes);
      tma_load_tile<D>(sK, &map_k, &sh.res_full, col0, h, b);
      tma_load_tile<D>(sV, &map_v, &sh.res_full, col0, h, b);
      for (int n = 0; n < nq; ++n) {
        const int s = n % kKvStages, q0 = (int)sh.subs[n] * 64;
        uint8_t* dst = ring + s * 2 * kSubBytes;
        if (!mbar_wait(&sh.ring_empty[s], ((n / kKvStages) & 1) ^ 1, abort_flag, status, 60)) break;
        mbar_expect_tx(&sh.ring_full[s], 2 * kSubBytes);
#pragma unroll
        for (int box = 0; box < Cfg::kBoxes; ++box) {
          tma_load_4d(dst + box * kSubBox, &map_q64, &sh.ring_full[s], box * 64, q0, h, b);
          tma_load_4d(dst + kSubBytes + box * kSubBox, &map_do64, &sh.ring_full[s], box * 64, q0, h, b);
        }
      }
    }
    __syncwarp();
  } else if (warp == kKvMmaWarp || warp == kKvMmaWarp + 1) {
    // Two issuing threads: one for the score products S^T and dP^T, one for the accumulating
    // products dV and dK.  The time a thread spends on its waits, commits and loop is in sequence
    // with the issue itself (which blocks while the tensor pipe is busy); split this way, one
    // thread's bookkeeping overlaps the other one's products.  Each barrier below has a single
    // waiting issuer, which sees every one of its phases.
    if (lane == 0 && tile_live) {
      const uint32_t k_addr = smem_u32(sK), v_addr = smem_u32(sV), ring_addr = smem_u32(ring);
      mbar_wait(&sh.res_full, 0, abort_flag, status, 61);
      if (warp == kKvMmaWarp) {
        // S^T and dP^T of sub-tile n into the buffers of group n & 1
        for (int n = 0; n < nq; ++n) {
          const int s = n % kKvStages, g = n & 1;
          const uint32_t q_addr = ring_addr + s * 2 * kSubBytes, do_addr = q_addr + kSubBytes;
          DQTRACE(true, n, 0);
          bool ok = mbar_wait(&sh.ring_full[s], (n / kKvStages) & 1, abort_flag, status, 62);
          DQTRACE(true, n, 1);
          // the buffers are free once dK of sub-tile n-2 has consumed dS^T (and dV before it P^T)
          if (n >= 2) ok = ok && mbar_wait(&sh.kd_done[g], ((n - 2) >> 1) & 1, abort_flag, status, 63);
          DQTRACE(true, n, 2);
          tc_fence_after_sync();
          if (ok) {
            issue_nt_n<D, FMT, 64>(tmem + g * 64, k_addr, Cfg::kBoxBytes, q_addr, kSubBox);         // S^T  = K . Q^T
            issue_nt_n<D, FMT, 64>(tmem + 128 + g * 64, v_addr, Cfg::kBoxBytes, do_addr, kSubBox);  // dP^T = V . dO^T
          }
          umma_commit(&sh.sdp_full[g]);
          DQTRACE(true, n, 3);
        }
        if (status) atomicAdd((unsigned long long*)(status + 4), (unsigned long long)nq);
      } else {
        for (int n = 0; n < nq; ++n) {
          const int s = n % kKvStages, g = n & 1;
          const uint32_t q_addr = ring_addr + s * 2 * kSubBytes, do_addr = q_addr + kSubBytes;
          DQTRACE(true, n, 4);
          bool ok = mbar_wait(&sh.p_full[g], (n >> 1) & 1, abort_flag, status, 64);
          DQTRACE(true, n, 5);
          tc_fence_after_sync();
          // query rows beyond the end of the sequence: padding rows of Q and dO stay out of the
          // reductions (the score products of this sub-tile have completed), see zero_tail_rows
          int nks = 4;
          const int valid = len - (int)sh.subs[n] * 64;
          if (ok && valid < 64) {
            uint8_t* stage = ring + s * 2 * kSubBytes;
            zero_tail_rows(stage, valid, Cfg::kBoxes, 64);
            nks = zero_tail_rows(stage + kSubBytes, valid, Cfg::kBoxes, 64);
          }
          if (ok) issue_tn_k<D, FMT, 64>(tmem_dv, tmem + g * 64, do_addr, kSubBox, n > 0, nks);          // dV += P^T . dO
          ok = ok && mbar_wait(&sh.ds_full[g], (n >> 1) & 1, abort_flag, status, 65);
          tc_fence_after_sync();
          if (ok) issue_tn_k<D, FMT, 64>(tmem_dk, tmem + 128 + g * 64, q_addr, kSubBox, n > 0, nks);     // dK += dS^T . Q
          umma_commit(&sh.kd_done[g]);
          umma_commit(&sh.ring_empty[s]);
          DQTRACE(true, n, 6);
        }
        umma_commit(&sh.acc_full);
        if (status) atomicAdd((unsigned long long*)(status + 4), (unsigned long long)nq);
      }
    }
    __syncwarp();
  } else {
    // Sixteen row warps: group g = sub-tiles of parity g, and inside a group two threads per key row,
    // thread half h taking query columns [32h, 32h+32) of a sub-tile.
    const int grp = (warp >> 2) & 1;
    const int half = warp >> 3;
    const int row = (warp & 3) * 32 + lane;
    const int gt = (half << 7) | row;            // thread index inside the group (0..255)
    const int j = col0 + row;
    const bool live = j < len;
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    // my 32 score columns; P^T / dS^T (16-bit pairs) go to the first 16 of them
    const uint32_t t_s = tmem + lane_base + grp * 64 + half * 32, t_dp = t_s + 128;
    const int64_t bhl = (int64_t)bh * L;
    if (tile_live) {
      const float c1 = p.scale * (MODE == ENTMAX ? (p.alpha - 1.f) : kLog2e);
      const float e = MODE == ENTMAX ? 1.f / (p.alpha - 1.f) : 0.f;
      const float* gstat = (MODE == ENTMAX ? p.tau : p.lse) + bhl;
      const float tau_head = MODE == LAZY ? p.tau_h[h] : 0.f;
      int k = 0;   // count of sub-tiles this group has handled
      for (int n = grp; n < nq; n += 2, ++k) {
        const int q0 = (int)sh.subs[n] * 64;
        float (*st)[64] = sh.stat[grp][k & 1];
        if (gt < 64) {   // stage the statistics of this sub-tile's 64 query rows
          const int qi = q0 + gt;
          const bool ql = qi < len;
          // entmax keeps the negated values: they are the addends of  x = s*c1 - tau  and  dP - delta
          const float sgn = MODE == ENTMAX ? -1.f : 1.f;
          st[0][gt] = ql ? sgn * gstat[qi] : 0.f;
          st[1][gt] = ql ? sgn * p.delta[bhl + qi] : 0.f;
          st[2][gt] = MODE == LAZY ? tau_head / (float)(qi + 1) : 0.f;
        }
        named_bar_sync(1 + grp, kKvGroupThreads);
        // query column c (row q0 + c) may use key j iff cmin <= c <= cmax
        const int cmax = live ? min(63, len - 1 - q0) : -1;
        const int cmin = causal ? j - q0 : 0;
        const bool need_mask = (causal && q0 < col0 + 128) || (q0 + 63 >= len) || (col0 + 127 >= len);
        const bool in_window = MODE == LAZY && (q0 - col0 - 127 < p.window);
        DQTRACE((tid & 127) == 0 && half == 0, n, 8);
        mbar_wait(&sh.sdp_full[grp], k & 1, abort_flag, status, 66);
        DQTRACE((tid & 127) == 0 && half == 0, n, 9);
        __syncwarp();
        tc_fence_after_sync();
        // 16 query columns at a time.  P^T chunk c lands in columns [8c, 8c+8) of this thread's part
        // of the S^T buffer and dS^T chunk c in the same columns of the dP^T buffer: both ranges were
        // read in an earlier or the same chunk, and belong to this thread alone.
#pragma unroll 1
        for (int ch = 0; ch < 2; ++ch) {
          uint32_t r[16], g32[16], pk[8], dk[8];
          tmem_ld16(t_s + ch * 16, r);
          tmem_ld16(t_dp + ch * 16, g32);
          tmem_ld_wait_regs16(r);
          tmem_ld_wait_regs16(g32);
          const int cb = half * 32 + ch * 16;        // first query column of this chunk
          const float* s0 = st[0] + cb;
          const float* s1 = st[1] + cb;
          const float* s2 = st[2] + cb;
          if (MODE == ENTMAX && KIND == 0 && !need_mask) {
            // alpha = 1.5, no masked entry: U = max(x, 0) by one saturating fma (x <= 1 everywhere),
            // P = U^2, dS = U (dP - delta) as packed pairs
#pragma unroll
            for (int x = 0; x < 16; x += 2) {
              const float e0 = __saturatef(fmaf(__uint_as_float(r[x]), c1, s0[x]));
              const float e1 = __saturatef(fmaf(__uint_as_float(r[x + 1]), c1, s0[x + 1]));
              const uint64_t ee = pack2(e0, e1);
              const uint64_t dd = add2(pack2(__uint_as_float(g32[x]), __uint_as_float(g32[x + 1])),
                                       *reinterpret_cast<const uint64_t*>(s1 + x));
              float p0, p1, d0, d1;
              unpack2(mul2(ee, ee), p0, p1);
              unpack2(mul2(ee, dd), d0, d1);
              pk[x >> 1] = pack16<FMT>(p0, p1);
              dk[x >> 1] = pack16<FMT>(d0, d1);
            }
          } else if (MODE == LAZY && !need_mask && !in_window) {
            // interior sub-tile: no masked entry and no bias, straight-line arithmetic
#pragma unroll
            for (int x = 0; x < 16; x += 2) {
              const float w0 = fast_exp2(fmaf(__uint_as_float(r[x]), c1, -s0[x]));
              const float w1 = fast_exp2(fmaf(__uint_as_float(r[x + 1]), c1, -s0[x + 1]));
              const float t0 = w0 + s2[x], t1 = w1 + s2[x + 1];
              const float md0 = t0 > 0.f ? __uint_as_float(g32[x]) : 0.f;
              const float md1 = t1 > 0.f ? __uint_as_float(g32[x + 1]) : 0.f;
              pk[x >> 1] = pack16<FMT>(fmaxf(t0, 0.f), fmaxf(t1, 0.f));
              dk[x >> 1] = pack16<FMT>(w0 * (md0 - s1[x]), w1 * (md1 - s1[x + 1]));
            }
          } else {
#pragma unroll
            for (int x = 0; x < 16; x += 2) {
              float pvv[2], dsv[2];
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
                  xs -= s0[x + y];
                }
                const bool valid = !need_mask || (c >= cmin && c <= cmax);
                float pv, w;
                bool m;
                prob_terms<MODE, KIND>(xs, e, s2[x + y], valid, pv, w, m);
                const float dp = __uint_as_float(g32[x + y]);
                pvv[y] = pv;
                // masked entries: exactly zero, whatever dP holds there (padding may be NaN)
                dsv[y] = MODE == ENTMAX ? (m ? w * (dp + s1[x + y]) : 0.f) : (valid ? w * ((m ? dp : 0.f) - s1[x + y]) : 0.f);
              }
              pk[x >> 1] = pack16<FMT>(pvv[0], pvv[1]);
              dk[x >> 1] = pack16<FMT>(dsv[0], dsv[1]);
            }
          }
          tmem_st8(t_s + ch * 8, pk);
          tmem_st8(t_dp + ch * 8, dk);
        }
        tmem_st_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(&sh.p_full[grp]);
          mbar_arrive(&sh.ds_full[grp]);
        }
        DQTRACE((tid & 127) == 0 && half == 0, n, 10);
      }
      mbar_wait(&sh.acc_full, 0, abort_flag, status, 67);   // (committed even when no sub-tile was visited)
      __syncwarp();
      tc_fence_after_sync();
      // group 0 stores dK, group 1 stores dV; the two threads of a row take half of the columns each
      uint8_t* grow = (uint8_t*)(grp == 0 ? p.dk.ptr : p.dv.ptr) +
                      2 * ((int64_t)b * (grp == 0 ? p.dk.s[0] : p.dv.s[0]) + (int64_t)h * (grp == 0 ? p.dk.s[1] : p.dv.s[1]) +
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
            uint4 w;
            w.x = (live && nq > 0) ? pack16<FMT>(__uint_as_float(o[x + 0]) * mul, __uint_as_float(o[x + 1]) * mul) : 0u;
            w.y = (live && nq > 0) ? pack16<FMT>(__uint_as_float(o[x + 2]) * mul, __uint_as_float(o[x + 3]) * mul) : 0u;
            w.z = (live && nq > 0) ? pack16<FMT>(__uint_as_float(o[x + 4]) * mul, __uint_as_float(o[x + 5]) * mul) : 0u;
            w.w = (live && nq > 0) ? pack16<FMT>(__uint_as_float(o[x + 6]) * mul, __uint_as_float(o[x + 7]) * mul) : 0u;
            *(uint4*)(grow + (ch * 32 + x) * 2) = w;
          }
        }
      }
    } else if (j < L) {
      uint8_t* grow = (uint8_t*)(grp == 0 ? p.dk.ptr : p.dv.ptr) +
                      2 * ((int64_t)b * (grp == 0 ? p.dk.s[0] : p.dv.s[0]) + (int64_t)h * (grp == 0 ? p.dk.s[1] : p.dv.s[1]) +
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
