// SIMT (CUDA-core, fp32 arithmetic) kernels for alpha-entmax attention and Lazy Attention.
//
// This family serves what the tensor-core family does not: fp32 inputs (the
// reference's tests check fp32 entmax outputs to 1e-4, which TF32/bf16 products
// cannot meet), head dims other than 64/128, unaligned strides.  It is also the
// on-device cross-check for the tensor-core kernels at sizes the CPU oracle
// cannot reach.  Tiles are 64 query rows x 64 keys, 256 threads; thread
// (ty, tx) = (tid/16, tid%16) owns rows ty*4..ty*4+3 and columns tx, tx+16,
// tx+32, tx+48 of a score tile, so a row lives in one half-warp.
//
// Forward replaces lazy_attention_triton.py:9-174 (LSE + output kernels) and the
// absent adasplash forward; backward replaces lazy_attention_triton.py:180-497.
#include "common.cuh"

namespace fla {
namespace simt {

constexpr int BM = 64;
constexpr int BN = 64;
constexpr int NT = 256;
constexpr int PLD = 65;  // leading dimension of the 64x64 probability tiles

__device__ __forceinline__ float half_warp_max(float x) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, o));
  return x;
}
__device__ __forceinline__ float half_warp_sum(float x) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}

// dst[r][d] = src row (row0 + r) if that row index < limit, else 0; columns D..DP-1 are 0.
template <typename T, int NDC>
__device__ __forceinline__ void load_tile(float* dst, const T* base, int64_t row_stride, int row0,
                                          int limit, int D) {
  constexpr int DP = NDC * 16, LD = DP + 1;
  for (int idx = threadIdx.x; idx < BM * DP; idx += NT) {
    int r = idx / DP, d = idx - r * DP;
    int row = row0 + r;
    float x = 0.f;
    if (row < limit && d < D) x = to_f32<T>(base[(int64_t)row * row_stride + d]);
    dst[r * LD + d] = x;
  }
}

// acc[a][b] = sum_d A[ty*4+a][d] * B[tx+16b][d]
template <int NDC>
__device__ __forceinline__ void gemm_nt(const float* As, const float* Bs, float acc[4][4], int ty, int tx) {
  constexpr int DP = NDC * 16, LD = DP + 1;
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int b = 0; b < 4; ++b) acc[a][b] = 0.f;
#pragma unroll 4
  for (int d = 0; d < DP; ++d) {
    float av[4], bv[4];
#pragma unroll
    for (int a = 0; a < 4; ++a) av[a] = As[(ty * 4 + a) * LD + d];
#pragma unroll
    for (int b = 0; b < 4; ++b) bv[b] = Bs[(tx + 16 * b) * LD + d];
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
      for (int b = 0; b < 4; ++b) acc[a][b] = fmaf(av[a], bv[b], acc[a][b]);
  }
}

// acc[a][c] += sum_k P[ty*4+a][k] * V[k][tx+16c]
template <int NDC>
__device__ __forceinline__ void gemm_nn_acc(const float* Ps, const float* Vs, float acc[4][NDC], int ty, int tx) {
  constexpr int LD = NDC * 16 + 1;
#pragma unroll 2
  for (int k = 0; k < BN; ++k) {
    float pv[4];
#pragma unroll
    for (int a = 0; a < 4; ++a) pv[a] = Ps[(ty * 4 + a) * PLD + k];
#pragma unroll
    for (int c = 0; c < NDC; ++c) {
      float vv = Vs[k * LD + tx + 16 * c];
#pragma unroll
      for (int a = 0; a < 4; ++a) acc[a][c] = fmaf(pv[a], vv, acc[a][c]);
    }
  }
}

// acc[a][c] += sum_q P[q][ty*4+a] * O[q][tx+16c]
template <int NDC>
__device__ __forceinline__ void gemm_tn_acc(const float* Ps, const float* Os, float acc[4][NDC], int ty, int tx) {
  constexpr int LD = NDC * 16 + 1;
#pragma unroll 2
  for (int q = 0; q < BM; ++q) {
    float pv[4];
#pragma unroll
    for (int a = 0; a < 4; ++a) pv[a] = Ps[q * PLD + ty * 4 + a];
#pragma unroll
    for (int c = 0; c < NDC; ++c) {
      float ov = Os[q * LD + tx + 16 * c];
#pragma unroll
      for (int a = 0; a < 4; ++a) acc[a][c] = fmaf(pv[a], ov, acc[a][c]);
    }
  }
}

// Score tile in the units the row statistics use: entmax X = (alpha-1) q.k/sqrt(D); lazy
// S log2(e) with S = q.k/sqrt(D) + bias[h, i-j] inside the window (the saved log-sum-exp is
// in the same base-2 units, so that every kernel forms exp2(x - lse) from identical terms).
// Entries that are not valid keys of their row are -inf.
template <int MODE, int NDC>
__device__ __forceinline__ void score_tile(const AttnParams& p, const float* Qs, const float* Ks, int h,
                                           int row0, int col0, int len, bool causal, int ty, int tx,
                                           float X[4][4]) {
  gemm_nt<NDC>(Qs, Ks, X, ty, tx);
  const float mul = MODE == ENTMAX ? p.scale * (p.alpha - 1.f) : p.scale * kLog2e;
#pragma unroll
  for (int a = 0; a < 4; ++a) {
    int i = row0 + ty * 4 + a;
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      int j = col0 + tx + 16 * b;
      float x = X[a][b] * mul;
      if (MODE == LAZY) {
        int dist = i - j;
        if (dist >= 0 && dist < p.window) x = fmaf(p.bias[(int64_t)h * p.bias_stride + dist], kLog2e, x);
      }
      bool valid = (j < len) && (!causal || j <= i);
      X[a][b] = valid ? x : -INFINITY;
    }
  }
}

template <typename T>
__device__ __forceinline__ const T* head_ptr(const View4& v, int b, int h) {
  return (const T*)v.ptr + (int64_t)b * v.s[0] + (int64_t)h * v.s[1];
}
template <typename T>
__device__ __forceinline__ T* head_ptr_mut(const View4& v, int b, int h) {
  return (T*)v.ptr + (int64_t)b * v.s[0] + (int64_t)h * v.s[1];
}

// ------------------------------------------------------------------------------------------
// Forward: row statistics (entmax: max + threshold iterations; lazy: log-sum-exp) followed by
// the output pass, one CTA per 64-row query tile.
// ------------------------------------------------------------------------------------------
template <int MODE, typename T, int NDC, int KIND>
__global__ void __launch_bounds__(NT) fwd_kernel(AttnParams p) {
  extern __shared__ float smem[];
  constexpr int DP = NDC * 16, LD = DP + 1;
  float* Qs = smem;
  float* Ks = Qs + BM * LD;
  float* Vs = Ks + BM * LD;
  float* Ps = Vs + BM * LD;
  float* Us = Ps + BM * PLD;
  float* Fs = Us + BM * PLD;  // lazy: the elastic probabilities before rounding to T

  const int mt = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  const int L = p.L, D = p.D;
  const int len = p.varlen ? min(max(p.varlen[b], 0), L) : L;
  const int row0 = mt * BM;
  const bool causal = (MODE == LAZY) ? true : (p.causal != 0);
  const int64_t bh = (int64_t)b * p.H + h;
  const bool want_aux = p.aux_o != nullptr;

  T* ob = head_ptr_mut<T>(p.o, b, h);
  float* stat = (MODE == ENTMAX ? p.tau : p.lse) + bh * L;

  if (row0 >= len) {  // whole tile is padding: zeros everywhere
    for (int idx = tid; idx < BM * D; idx += NT) {
      int r = idx / D, d = idx - r * D;
      if (row0 + r < L) {
        ob[(int64_t)(row0 + r) * p.o.s[2] + d] = from_f32<T>(0.f);
        if (want_aux) {
          if (MODE == ENTMAX) p.aux_o[(bh * L + row0 + r) * D + d] = 0.f;
          else { p.aux_o[(bh * L + row0 + r) * 2 * D + d] = 0.f; p.aux_o[(bh * L + row0 + r) * 2 * D + D + d] = 0.f; }
        }
      }
    }
    if (tid < BM && row0 + tid < L) {
      stat[row0 + tid] = 0.f;
      if (MODE == ENTMAX && p.aux_s) p.aux_s[bh * L + row0 + tid] = 0.f;
    }
    return;
  }

  const T* qb = head_ptr<T>(p.q, b, h);
  const T* kb = head_ptr<T>(p.k, b, h);
  const T* vb = head_ptr<T>(p.v, b, h);
  const int kend = causal ? min(len, row0 + BM) : len;
  const int nkt = (kend + BN - 1) / BN;

  load_tile<T, NDC>(Qs, qb, p.q.s[2], row0, len, D);

  float X[4][4];
  float rstat[4];  // tau (entmax, absolute) or lse (lazy) per owned row

  if (MODE == ENTMAX) {
    const float e = 1.f / (p.alpha - 1.f);
    float m[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
    for (int kt = 0; kt < nkt; ++kt) {
      __syncthreads();
      load_tile<T, NDC>(Ks, kb, p.k.s[2], kt * BN, len, D);
      __syncthreads();
      score_tile<MODE, NDC>(p, Qs, Ks, h, row0, kt * BN, len, causal, ty, tx, X);
#pragma unroll
      for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int c = 0; c < 4; ++c) m[a] = fmaxf(m[a], X[a][c]);
    }
    float ts[4], lo[4], hi[4];
    bool done[4];
#pragma unroll
    for (int a = 0; a < 4; ++a) {
      m[a] = half_warp_max(m[a]);
      int i = row0 + ty * 4 + a;
      float n = (float)(causal ? min(i + 1, len) : len);
      lo[a] = -1.f;
      hi[a] = -exp2f(-(p.alpha - 1.f) * log2f(n));
      ts[a] = -1.f;  // left end of the bracket: iterations increase monotonically
      done[a] = (i >= len) || (n <= 1.f);
      if (n <= 1.f) ts[a] = -1.f;  // a single valid key: p = 1 exactly
    }
    for (int it = 0; it < p.niter; ++it) {
      float s0[4] = {0, 0, 0, 0}, s1[4] = {0, 0, 0, 0}, s2[4] = {0, 0, 0, 0};
      for (int kt = 0; kt < nkt; ++kt) {
        __syncthreads();
        load_tile<T, NDC>(Ks, kb, p.k.s[2], kt * BN, len, D);
        __syncthreads();
        score_tile<MODE, NDC>(p, Qs, Ks, h, row0, kt * BN, len, causal, ty, tx, X);
#pragma unroll
        for (int a = 0; a < 4; ++a)
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            float d = (X[a][c] - m[a]) - ts[a];
            if (d > 0.f) {  // -inf entries never pass
              float pw, u;
              p_and_u<KIND>(d, e, pw, u);
              s0[a] += pw;
              s1[a] += u;
              s2[a] += (KIND == 0) ? 1.f : ((KIND == 1) ? 0.f : u / d);
            }
          }
      }
      bool all_done = true;
#pragma unroll
      for (int a = 0; a < 4; ++a) {
        float r0 = half_warp_sum(s0[a]), r1 = half_warp_sum(s1[a]), r2 = half_warp_sum(s2[a]);
        if (!done[a]) {
          float t = tau_update(ts[a], r0, r1, r2, e, lo[a], hi[a]);
          if (fabsf(t - ts[a]) <= 1.2e-7f) done[a] = true;
          ts[a] = t;
        }
        all_done = all_done && done[a];
      }
      if (__syncthreads_and(all_done)) break;
    }
#pragma unroll
    for (int a = 0; a < 4; ++a) rstat[a] = m[a] + ts[a];
  } else {
    float m[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
    for (int kt = 0; kt < nkt; ++kt) {
      __syncthreads();
      load_tile<T, NDC>(Ks, kb, p.k.s[2], kt * BN, len, D);
      __syncthreads();
      score_tile<MODE, NDC>(p, Qs, Ks, h, row0, kt * BN, len, causal, ty, tx, X);
#pragma unroll
      for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int c = 0; c < 4; ++c) m[a] = fmaxf(m[a], X[a][c]);
    }
    float l[4] = {0, 0, 0, 0};
#pragma unroll
    for (int a = 0; a < 4; ++a) m[a] = half_warp_max(m[a]);
    for (int kt = 0; kt < nkt; ++kt) {
      __syncthreads();
      load_tile<T, NDC>(Ks, kb, p.k.s[2], kt * BN, len, D);
      __syncthreads();
      score_tile<MODE, NDC>(p, Qs, Ks, h, row0, kt * BN, len, causal, ty, tx, X);
#pragma unroll
      for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int c = 0; c < 4; ++c)
          if (X[a][c] > -INFINITY) l[a] += exp2f(X[a][c] - m[a]);
    }
#pragma unroll
    for (int a = 0; a < 4; ++a) rstat[a] = m[a] + log2f(half_warp_sum(l[a]));
  }

  // ---- output pass -------------------------------------------------------------------------
  float acc_o[4][NDC], acc_u[4][NDC], acc_f[4][NDC];
  float su[4] = {0, 0, 0, 0};
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int c = 0; c < NDC; ++c) { acc_o[a][c] = 0.f; acc_u[a][c] = 0.f; acc_f[a][c] = 0.f; }
  const float e = MODE == ENTMAX ? 1.f / (p.alpha - 1.f) : 0.f;
  const float tau_head = MODE == LAZY ? p.tau_h[h] : 0.f;

  for (int kt = 0; kt < nkt; ++kt) {
    __syncthreads();
    load_tile<T, NDC>(Ks, kb, p.k.s[2], kt * BN, len, D);
    load_tile<T, NDC>(Vs, vb, p.v.s[2], kt * BN, len, D);
    __syncthreads();
    score_tile<MODE, NDC>(p, Qs, Ks, h, row0, kt * BN, len, causal, ty, tx, X);
    int any_nz = 0;
#pragma unroll
    for (int a = 0; a < 4; ++a) {
      int i = row0 + ty * 4 + a;
      bool live = i < len;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        float pw = 0.f, u = 0.f;
        if (MODE == ENTMAX) {
          float d = X[a][c] - rstat[a];
          if (live && d > 0.f) p_and_u<KIND>(d, e, pw, u);
        } else {
          if (live && X[a][c] > -INFINITY) {
            float t = exp2f(X[a][c] - rstat[a]) + tau_head / (float)(i + 1);
            if (t > 0.f) { pw = t; u = 1.f; }
          }
        }
        any_nz |= (pw > 0.f);
        su[a] += u;
        Ps[(ty * 4 + a) * PLD + tx + 16 * c] = round_to<T>(pw);
        Us[(ty * 4 + a) * PLD + tx + 16 * c] = u;
        if (MODE == LAZY) Fs[(ty * 4 + a) * PLD + tx + 16 * c] = pw;
      }
    }
    int tile_nz = __syncthreads_or(any_nz);
    if (MODE == ENTMAX && p.block_mask && tile_nz && tid == 0) {
      uint32_t* w = p.block_mask + ((bh * ((L + 127) / 128) + (row0 >> 7)) * p.mask_words) + (kt >> 5);
      atomicOr(w, 1u << (kt & 31));
    }
    gemm_nn_acc<NDC>(Ps, Vs, acc_o, ty, tx);
    if (want_aux) gemm_nn_acc<NDC>(Us, Vs, acc_u, ty, tx);
    if (MODE == LAZY && want_aux) gemm_nn_acc<NDC>(Fs, Vs, acc_f, ty, tx);
  }

#pragma unroll
  for (int a = 0; a < 4; ++a) {
    int i = row0 + ty * 4 + a;
    if (i >= L) continue;
    bool live = i < len;
    float s_u = half_warp_sum(su[a]);
#pragma unroll
    for (int c = 0; c < NDC; ++c) {
      int d = tx + 16 * c;
      if (d < D) {
        ob[(int64_t)i * p.o.s[2] + d] = from_f32<T>(live ? acc_o[a][c] : 0.f);
        if (want_aux) {
          if (MODE == ENTMAX) p.aux_o[(bh * L + i) * D + d] = live ? acc_u[a][c] : 0.f;
          else {
            p.aux_o[(bh * L + i) * 2 * D + d] = live ? acc_f[a][c] : 0.f;
            p.aux_o[(bh * L + i) * 2 * D + D + d] = live ? acc_u[a][c] : 0.f;
          }
        }
      }
    }
    if (tx == 0) {
      stat[i] = live ? rstat[a] : 0.f;
      if (MODE == ENTMAX && p.aux_s) p.aux_s[bh * L + i] = live ? s_u : 0.f;
    }
  }
}

// ------------------------------------------------------------------------------------------
// Row pre-pass of the backward, one warp per query row (shared by both kernel families):
//   entmax: delta_i = dO_i . (U V)_i / sum_j U_ij
//   lazy:   r_i = dO_i . (M V)_i,  delta_i = dO_i . O_i - tau_h/(i+1) r_i,  dtau_h += r_i/(i+1)
//           (O_i in fp32 and (M V)_i are the two halves of the row's aux record)
// (replaces the O(L^2 D) recompute pre-pass lazy_attention_triton.py:180-270).
// ------------------------------------------------------------------------------------------
template <int MODE, typename T>
__global__ void __launch_bounds__(256) delta_kernel(AttnParams p) {
  __shared__ float s_dtau[8];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int i = blockIdx.x * 8 + warp, h = blockIdx.y, b = blockIdx.z;
  const int L = p.L, D = p.D;
  const int len = p.varlen ? min(max(p.varlen[b], 0), L) : L;
  const int64_t bh = (int64_t)b * p.H + h;
  float contrib = 0.f;
  if (i < L) {
    float delta = 0.f;
    if (i < len) {
      const T* dob = head_ptr<T>(p.dout, b, h) + (int64_t)i * p.dout.s[2];
      const float* ax = p.aux_o + (bh * L + i) * (MODE == ENTMAX ? D : 2 * D);
      float r = 0.f, oo = 0.f;
      for (int d = lane; d < D; d += 32) {
        float g = to_f32<T>(dob[d]);
        if (MODE == ENTMAX) r = fmaf(g, ax[d], r);
        else { oo = fmaf(g, ax[d], oo); r = fmaf(g, ax[D + d], r); }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        r += __shfl_xor_sync(0xffffffffu, r, o);
        oo += __shfl_xor_sync(0xffffffffu, oo, o);
      }
      if (MODE == ENTMAX) {
        float s = p.aux_s[bh * L + i];
        delta = s > 0.f ? r / s : 0.f;
      } else {
        float inv = 1.f / (float)(i + 1);
        delta = oo - p.tau_h[h] * inv * r;
        contrib = r * inv;
      }
    }
    if (lane == 0) p.delta[bh * L + i] = delta;
  }
  if (MODE == LAZY && p.dtau_acc != nullptr) {
    if (lane == 0) s_dtau[warp] = contrib;
    __syncthreads();
    if (threadIdx.x == 0) {
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < 8; ++w) s += s_dtau[w];
      if (s != 0.f) atomicAdd(p.dtau_acc + h, to_fixed(s));
    }
  }
}

// dS for one score entry.  stat = tau (entmax) / lse (lazy).  Also returns the probability
// that multiplies dO in dV (P for entmax, the elastic A for lazy).
template <int MODE, int KIND>
__device__ __forceinline__ void ds_entry(float x, float stat, float delta, float dA, float e, float tau_head,
                                         int i, bool live, float& pv, float& ds) {
  pv = 0.f;
  ds = 0.f;
  if (!live || !(x > -INFINITY)) return;
  if (MODE == ENTMAX) {
    float d = x - stat;
    if (d > 0.f) {
      float u;
      p_and_u<KIND>(d, e, pv, u);
      ds = u * (dA - delta);
    }
  } else {
    float pn = exp2f(x - stat);
    float t = pn + tau_head / (float)(i + 1);
    bool m = t > 0.f;
    pv = m ? t : 0.f;
    ds = pn * ((m ? dA : 0.f) - delta);
  }
}

// ------------------------------------------------------------------------------------------
// dQ (and dbias for lazy): one CTA per 64-row query tile, streams key tiles.
// ------------------------------------------------------------------------------------------
template <int MODE, typename T, int NDC, int KIND>
__global__ void __launch_bounds__(NT) dq_kernel(AttnParams p) {
  extern __shared__ float smem[];
  constexpr int DP = NDC * 16, LD = DP + 1;
  float* Qs = smem;
  float* dOs = Qs + BM * LD;
  float* Ks = dOs + BM * LD;
  float* Vs = Ks + BM * LD;
  float* dSs = Vs + BM * LD;
  __shared__ unsigned long long diag[128];  // per-tile sums over the diagonals i-j, fixed point (see to_fixed)

  const int mt = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  const int L = p.L, D = p.D;
  const int len = p.varlen ? min(max(p.varlen[b], 0), L) : L;
  const int row0 = mt * BM;
  const bool causal = (MODE == LAZY) ? true : (p.causal != 0);
  const int64_t bh = (int64_t)b * p.H + h;
  T* dqb = head_ptr_mut<T>(p.dq, b, h);

  if (row0 >= len) {
    for (int idx = tid; idx < BM * D; idx += NT) {
      int r = idx / D, d = idx - r * D;
      if (row0 + r < L) dqb[(int64_t)(row0 + r) * p.dq.s[2] + d] = from_f32<T>(0.f);
    }
    return;
  }
  const T* kb = head_ptr<T>(p.k, b, h);
  const T* vb = head_ptr<T>(p.v, b, h);
  load_tile<T, NDC>(Qs, head_ptr<T>(p.q, b, h), p.q.s[2], row0, len, D);
  load_tile<T, NDC>(dOs, head_ptr<T>(p.dout, b, h), p.dout.s[2], row0, len, D);

  const float* stat = (MODE == ENTMAX ? p.tau : p.lse) + bh * L;
  float rstat[4], rdelta[4];
#pragma unroll
  for (int a = 0; a < 4; ++a) {
    int i = row0 + ty * 4 + a;
    rstat[a] = i < len ? stat[i] : 0.f;
    rdelta[a] = i < len ? p.delta[bh * L + i] : 0.f;
  }
  const float e = MODE == ENTMAX ? 1.f / (p.alpha - 1.f) : 0.f;
  const float tau_head = MODE == LAZY ? p.tau_h[h] : 0.f;
  const bool want_dbias = MODE == LAZY && p.dbias_acc != nullptr;

  float acc[4][NDC];
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int c = 0; c < NDC; ++c) acc[a][c] = 0.f;

  const int kend = causal ? min(len, row0 + BM) : len;
  const int nkt = (kend + BN - 1) / BN;
  float X[4][4], dA[4][4];
  for (int kt = 0; kt < nkt; ++kt) {
    __syncthreads();
    load_tile<T, NDC>(Ks, kb, p.k.s[2], kt * BN, len, D);
    load_tile<T, NDC>(Vs, vb, p.v.s[2], kt * BN, len, D);
    if (want_dbias && tid < 128) diag[tid] = 0ull;
    __syncthreads();
    score_tile<MODE, NDC>(p, Qs, Ks, h, row0, kt * BN, len, causal, ty, tx, X);
    gemm_nt<NDC>(dOs, Vs, dA, ty, tx);
    // distances covered by this tile: (row0 - col0) - 63 .. (row0 - col0) + 63
    const int dbase = row0 - kt * BN - 63;
    const bool tile_in_window = want_dbias && (dbase < p.window) && (dbase + 126 >= 0);
#pragma unroll
    for (int a = 0; a < 4; ++a) {
      int i = row0 + ty * 4 + a;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        float pv, ds;
        ds_entry<MODE, KIND>(X[a][c], rstat[a], rdelta[a], dA[a][c], e, tau_head, i, i < len, pv, ds);
        dSs[(ty * 4 + a) * PLD + tx + 16 * c] = round_to<T>(ds);
        if (tile_in_window && ds != 0.f) {
          int j = kt * BN + tx + 16 * c;
          atomicAdd(&diag[i - j - dbase], to_fixed(ds));
        }
      }
    }
    __syncthreads();
    gemm_nn_acc<NDC>(dSs, Ks, acc, ty, tx);
    if (tile_in_window && tid < 127) {
      int w = dbase + tid;
      const unsigned long long s = diag[tid];
      if (w >= 0 && w < p.window && s != 0ull) atomicAdd(p.dbias_acc + (int64_t)h * p.dbias_acc_stride + w, s);
    }
  }
#pragma unroll
  for (int a = 0; a < 4; ++a) {
    int i = row0 + ty * 4 + a;
    if (i >= L) continue;
#pragma unroll
    for (int c = 0; c < NDC; ++c) {
      int d = tx + 16 * c;
      if (d < D) dqb[(int64_t)i * p.dq.s[2] + d] = from_f32<T>(i < len ? acc[a][c] * p.scale : 0.f);
    }
  }
}

// ------------------------------------------------------------------------------------------
// dK, dV: one CTA per 64-key tile, streams query tiles.
// ------------------------------------------------------------------------------------------
template <int MODE, typename T, int NDC, int KIND>
__global__ void __launch_bounds__(NT) dkdv_kernel(AttnParams p) {
  extern __shared__ float smem[];
  constexpr int DP = NDC * 16, LD = DP + 1;
  float* Ks = smem;
  float* Vs = Ks + BM * LD;
  float* Qs = Vs + BM * LD;
  float* dOs = Qs + BM * LD;
  float* Ps = dOs + BM * LD;
  float* dSs = Ps + BM * PLD;

  const int nt = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  const int L = p.L, D = p.D;
  const int len = p.varlen ? min(max(p.varlen[b], 0), L) : L;
  const int col0 = nt * BN;
  const bool causal = (MODE == LAZY) ? true : (p.causal != 0);
  const int64_t bh = (int64_t)b * p.H + h;
  T* dkb = head_ptr_mut<T>(p.dk, b, h);
  T* dvb = head_ptr_mut<T>(p.dv, b, h);

  if (col0 >= len) {
    for (int idx = tid; idx < BN * D; idx += NT) {
      int r = idx / D, d = idx - r * D;
      if (col0 + r < L) {
        dkb[(int64_t)(col0 + r) * p.dk.s[2] + d] = from_f32<T>(0.f);
        dvb[(int64_t)(col0 + r) * p.dv.s[2] + d] = from_f32<T>(0.f);
      }
    }
    return;
  }
  const T* qb = head_ptr<T>(p.q, b, h);
  const T* dob = head_ptr<T>(p.dout, b, h);
  load_tile<T, NDC>(Ks, head_ptr<T>(p.k, b, h), p.k.s[2], col0, len, D);
  load_tile<T, NDC>(Vs, head_ptr<T>(p.v, b, h), p.v.s[2], col0, len, D);

  const float* stat = (MODE == ENTMAX ? p.tau : p.lse) + bh * L;
  const float e = MODE == ENTMAX ? 1.f / (p.alpha - 1.f) : 0.f;
  const float tau_head = MODE == LAZY ? p.tau_h[h] : 0.f;

  float acc_k[4][NDC], acc_v[4][NDC];
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int c = 0; c < NDC; ++c) { acc_k[a][c] = 0.f; acc_v[a][c] = 0.f; }

  const int mt_begin = causal ? nt : 0;
  const int mt_end = (len + BM - 1) / BM;
  float X[4][4], dA[4][4];
  for (int mt = mt_begin; mt < mt_end; ++mt) {
    const int row0 = mt * BM;
    __syncthreads();
    load_tile<T, NDC>(Qs, qb, p.q.s[2], row0, len, D);
    load_tile<T, NDC>(dOs, dob, p.dout.s[2], row0, len, D);
    __syncthreads();
    score_tile<MODE, NDC>(p, Qs, Ks, h, row0, col0, len, causal, ty, tx, X);
    gemm_nt<NDC>(dOs, Vs, dA, ty, tx);
#pragma unroll
    for (int a = 0; a < 4; ++a) {
      int i = row0 + ty * 4 + a;
      bool live = i < len;
      float st = live ? stat[i] : 0.f;
      float dl = live ? p.delta[bh * L + i] : 0.f;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        float pv, ds;
        ds_entry<MODE, KIND>(X[a][c], st, dl, dA[a][c], e, tau_head, i, live, pv, ds);
        Ps[(ty * 4 + a) * PLD + tx + 16 * c] = round_to<T>(pv);
        dSs[(ty * 4 + a) * PLD + tx + 16 * c] = round_to<T>(ds);
      }
    }
    __syncthreads();
    gemm_tn_acc<NDC>(Ps, dOs, acc_v, ty, tx);
    gemm_tn_acc<NDC>(dSs, Qs, acc_k, ty, tx);
  }
#pragma unroll
  for (int a = 0; a < 4; ++a) {
    int j = col0 + ty * 4 + a;
    if (j >= L) continue;
    bool live = j < len;
#pragma unroll
    for (int c = 0; c < NDC; ++c) {
      int d = tx + 16 * c;
      if (d < D) {
        dkb[(int64_t)j * p.dk.s[2] + d] = from_f32<T>(live ? acc_k[a][c] * p.scale : 0.f);
        dvb[(int64_t)j * p.dv.s[2] + d] = from_f32<T>(live ? acc_v[a][c] : 0.f);
      }
    }
  }
}

// ------------------------------------------------------------------------------------------
// Host-side dispatch
// ------------------------------------------------------------------------------------------
template <int NDC>
constexpr size_t fwd_smem() { return sizeof(float) * (3 * BM * (NDC * 16 + 1) + 3 * BM * PLD); }
template <int NDC>
constexpr size_t dq_smem() { return sizeof(float) * (4 * BM * (NDC * 16 + 1) + BM * PLD + 128); }
template <int NDC>
constexpr size_t dkdv_smem() { return sizeof(float) * (4 * BM * (NDC * 16 + 1) + 2 * BM * PLD); }

template <typename K>
static cudaError_t set_smem(K kernel, size_t bytes) {
  return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
}

template <int MODE, typename T, int NDC, int KIND>
static cudaError_t launch_fwd_t(const AttnParams& p, cudaStream_t st) {
  auto kern = fwd_kernel<MODE, T, NDC, KIND>;
  cudaError_t err = set_smem(kern, fwd_smem<NDC>());
  if (err != cudaSuccess) return err;
  dim3 grid((p.L + BM - 1) / BM, p.H, p.B);
  kern<<<grid, NT, fwd_smem<NDC>(), st>>>(p);
  return cudaGetLastError();
}

template <int MODE, typename T, int NDC, int KIND>
static cudaError_t launch_bwd_t(const AttnParams& p, cudaStream_t st) {
  auto kq = dq_kernel<MODE, T, NDC, KIND>;
  auto kkv = dkdv_kernel<MODE, T, NDC, KIND>;
  cudaError_t err = set_smem(kq, dq_smem<NDC>());
  if (err != cudaSuccess) return err;
  err = set_smem(kkv, dkdv_smem<NDC>());
  if (err != cudaSuccess) return err;
  dim3 grid((p.L + BM - 1) / BM, p.H, p.B);
  kq<<<grid, NT, dq_smem<NDC>(), st>>>(p);
  err = cudaGetLastError();
  if (err != cudaSuccess) return err;
  kkv<<<grid, NT, dkdv_smem<NDC>(), st>>>(p);
  return cudaGetLastError();
}

template <int MODE, typename T, int NDC>
static cudaError_t launch_kind(const AttnParams& p, bool bwd, cudaStream_t st) {
  int kind = MODE == ENTMAX ? alpha_kind(p.alpha) : 0;
  if (MODE == LAZY || kind == 0) return bwd ? launch_bwd_t<MODE, T, NDC, 0>(p, st) : launch_fwd_t<MODE, T, NDC, 0>(p, st);
  if (kind == 1) return bwd ? launch_bwd_t<MODE, T, NDC, 1>(p, st) : launch_fwd_t<MODE, T, NDC, 1>(p, st);
  return bwd ? launch_bwd_t<MODE, T, NDC, 2>(p, st) : launch_fwd_t<MODE, T, NDC, 2>(p, st);
}

template <int MODE, typename T>
static cudaError_t launch_ndc(const AttnParams& p, bool bwd, cudaStream_t st) {
  if (p.D <= 16) return launch_kind<MODE, T, 1>(p, bwd, st);
  if (p.D <= 32) return launch_kind<MODE, T, 2>(p, bwd, st);
  if (p.D <= 64) return launch_kind<MODE, T, 4>(p, bwd, st);
  return launch_kind<MODE, T, 8>(p, bwd, st);
}

template <int MODE>
static cudaError_t launch_dtype(const AttnParams& p, int dtype, bool bwd, cudaStream_t st) {
  if (dtype == FLA_F32) return launch_ndc<MODE, float>(p, bwd, st);
  if (dtype == FLA_F16) return launch_ndc<MODE, __half>(p, bwd, st);
  return launch_ndc<MODE, __nv_bfloat16>(p, bwd, st);
}

}  // namespace simt

cudaError_t simt_attn_fwd(int mode, const AttnParams& p, int dtype, cudaStream_t st) {
  return mode == ENTMAX ? simt::launch_dtype<ENTMAX>(p, dtype, false, st)
                        : simt::launch_dtype<LAZY>(p, dtype, false, st);
}

cudaError_t simt_attn_bwd(int mode, const AttnParams& p, int dtype, cudaStream_t st) {
  return mode == ENTMAX ? simt::launch_dtype<ENTMAX>(p, dtype, true, st)
                        : simt::launch_dtype<LAZY>(p, dtype, true, st);
}

// Last step of a Lazy Attention backward with trained parameters: the fixed-point accumulators become the fp32
// gradients (columns of dbias at or beyond L cannot be reached by any distance i - j and are zero).
__global__ void lazy_params_finish_kernel(AttnParams p) {
  const int h = blockIdx.y;
  const int w = blockIdx.x * blockDim.x + threadIdx.x;
  const double inv = 1.0 / (double)kFixedScale;
  if (p.dbias != nullptr && w < p.window) {
    const long long a = w < p.dbias_acc_stride ? (long long)p.dbias_acc[(int64_t)h * p.dbias_acc_stride + w] : 0ll;
    p.dbias[(int64_t)h * p.dbias_stride + w] = (float)((double)a * inv);
  }
  if (p.dtau != nullptr && w == 0) p.dtau[h] = (float)((double)(long long)p.dtau_acc[h] * inv);
}

cudaError_t lazy_params_finish(const AttnParams& p, cudaStream_t st) {
  dim3 grid((max(p.window, 1) + 255) / 256, p.H);
  lazy_params_finish_kernel<<<grid, 256, 0, st>>>(p);
  return cudaGetLastError();
}

// Row pre-pass of the backward; used by both kernel families.
cudaError_t attn_delta(int mode, const AttnParams& p, int dtype, cudaStream_t st) {
  dim3 grid((p.L + 7) / 8, p.H, p.B);
#define FLA_DELTA(M, T) simt::delta_kernel<M, T><<<grid, 256, 0, st>>>(p)
  if (mode == ENTMAX) {
    if (dtype == FLA_F32) FLA_DELTA(ENTMAX, float);
    else if (dtype == FLA_F16) FLA_DELTA(ENTMAX, __half);
    else FLA_DELTA(ENTMAX, __nv_bfloat16);
  } else {
    if (dtype == FLA_F32) FLA_DELTA(LAZY, float);
    else if (dtype == FLA_F16) FLA_DELTA(LAZY, __half);
    else FLA_DELTA(LAZY, __nv_bfloat16);
  }
#undef FLA_DELTA
  return cudaGetLastError();
}

}  // namespace fla
